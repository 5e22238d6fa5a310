"""INT8 mixed-precision training: bf16 weights, dynamically quantized INT8 matmuls for the
forward, grad-input and grad-weight GEMMs (reference: subclasses/mixed_precision.py).

`MixedPrecisionConfig`, `MixedPrecisionLinearWeight`, `convert_mixed_precision` keep the
reference's names and semantics. Differences are in how the work is issued, not in its result:
  * every quantize is one sm_100a kernel, and a transposed operand is quantized by the
    transposing kernel instead of quantize-then-`.contiguous()`;
  * the forward's row-wise pass over the activation also records its per-column absmax, which
    the backward's grad-weight quantize reuses (one fewer pass over the activation);
  * under FSDP2 the weight shard is quantized before the all-gather (`fsdp_pre_all_gather`), so
    the gather moves int8 + one scale per row instead of bf16.
"""
from __future__ import annotations

from typing import Any, NamedTuple, Optional, Tuple

import torch
import torch.nn.functional as F
import torch.utils._pytree as pytree
from torch import Tensor, nn

import gn_kernels
from gn_kernels import scaled_mm

from .int8 import _quant_cache, _rows_quantize

aten = torch.ops.aten


class MixedPrecisionConfig(NamedTuple):
    output: bool = True
    grad_input: bool = True
    grad_weight: bool = True
    dtype: str = "int8"
    stochastic_rounding: bool = False


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


class MixedPrecisionLinearWeight(Tensor):
    """A bf16 weight whose `F.linear` runs INT8 matmuls (reference: mixed_precision.py:23-97)."""

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, data: Tensor, config: MixedPrecisionConfig):
        return Tensor._make_wrapper_subclass(cls, data.shape, dtype=data.dtype, device=data.device)

    @torch._dynamo.disable
    def __init__(self, data: Tensor, config: MixedPrecisionConfig):
        self._data = data
        self.config = config

    def __tensor_flatten__(self):
        return ["_data"], [self.config]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["_data"], *tensor_attributes)

    def __repr__(self):
        return f"{self.__class__.__name__}(data={self._data}, config={self.config})"

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or dict()
        if func is F.linear:
            return _Int8MixedPrecisionLinear.apply(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = kwargs or {}
        seen: list[MixedPrecisionConfig] = []

        def unwrap(x):
            if seen:
                assert x.config == seen[0]
            else:
                seen.append(x.config)
            return x._data

        out = func(*pytree.tree_map_only(cls, unwrap, args), **pytree.tree_map_only(cls, unwrap, kwargs))
        if func is aten.copy_.default:
            return args[0]
        if func in _REWRAP_OPS:
            return pytree.tree_map_only(Tensor, lambda t: cls(t, seen[0]), out)
        return out

    # ---- FSDP2 all-gather extension: gather int8 + scales instead of bf16 ------------------------
    # (the reference gathers this subclass in bf16; the hooks follow the protocol its BitNet
    # subclass uses, subclasses/bitnet.py:83-107)
    #
    # Forward gather: each rank quantizes its rows row-wise; rows of the gathered int8 weight are then
    # bit-identical to quantizing the whole weight (what the forward product needs).
    # Backward gather (FSDP2 gathers again when the parameters were resharded after forward): the
    # grad-input product needs the weight quantized along its OUTPUT dimension, which spans the ranks.
    # Ranks agree on the per-column maxima with one all-reduce(MAX) of a [K] vector (exact: max is
    # associative), quantize their rows with them, and the gathered int8 rows are again bit-identical to the
    # unsharded quantization; the [K] column scales are the same on every rank and are not gathered.
    # `backward_gather = "row"` keeps the forward's form for backward too (the weight's row scales are then
    # folded into dY, different rounding from the reference's): needed with activation checkpointing, whose
    # recomputed forward runs on the backward gather.
    backward_gather = "col"

    def fsdp_pre_all_gather(self, mesh, outer_size=None, outer_stride=None, module=None, mp_policy=None):
        cfg = self.config
        # INT8 rows serve the forward and the grad-input products; if either of them is configured to stay
        # in bf16 the reference computes it from the bf16 weight, so the bf16 weight is what gets gathered
        if cfg.dtype != "int8" or not (cfg.output and cfg.grad_input):
            return (self._data,), (None, None, None)
        # a mesh of one rank moves nothing, and FSDP2 then takes only the first tensor a hook returns
        if mesh is not None and mesh.size() == 1:
            return (self._data,), (None, None, None)
        in_backward = torch._C._current_graph_task_id() != -1
        if in_backward and type(self).backward_gather == "col":
            colmax = gn_kernels.col_absmax(self._data)
            group = mesh.get_group() if mesh is not None else None
            if torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
                torch.distributed.all_reduce(colmax, op=torch.distributed.ReduceOp.MAX, group=group)
            w_i8, col_scale = gn_kernels.quantize_colwise(self._data, colmax, torch.int8, cfg.stochastic_rounding)
            # the slot of the row scales keeps its size (FSDP2 sized the gather buffers in forward); its content is unused
            unused = self._data.new_empty((self._data.shape[0], 1))
            return (w_i8, unused), (cfg, "col", col_scale)
        w_i8, w_scale = gn_kernels.quantize_rowwise(self._data, torch.int8, cfg.stochastic_rounding)
        return (w_i8, w_scale), (cfg, "row", None)

    def fsdp_post_all_gather(self, all_gather_outputs: Tuple[Tensor, ...], metadata: Any, param_dtype: torch.dtype, *,
                             out: Optional[Tensor] = None):
        config, mode, col_scale = metadata
        if config is None:
            (data,) = all_gather_outputs
            if out is not None:
                return
            return MixedPrecisionLinearWeight(data, self.config), all_gather_outputs
        w_i8, w_scale = all_gather_outputs
        if out is not None:
            # the gather refilled the tensors `out` wraps; only what they mean may have changed
            assert isinstance(out, Int8RowScaledLinearWeight)
            out.mode, out.col_scale = mode, col_scale
            return
        return Int8RowScaledLinearWeight(w_i8, w_scale.view(-1, 1), config, mode, col_scale), all_gather_outputs


def _dynamic_int8_mm(A: Tensor, B: Tensor, sr: bool, *, a_col_absmax: Tensor | None = None,
                     b_col_absmax: Tensor | None = None, cache_a: bool = False, transposed_out: bool = False) -> Tensor:
    """bf16 A [M,K] @ B [K,N] through INT8: rows of A and columns of B get absmax scales
    (reference: mixed_precision.py:100-108). Either operand may be a transposed view; the optional
    absmax tensors are precomputed per-column maxima of the operand's BASE (row-major) tensor.
    `transposed_out` returns the contiguous transpose [N,M] of the same product (same bits)."""
    A_i8, row_scale = _rows_quantize(A, sr, 1e-12, col_absmax=a_col_absmax, cache=cache_a)
    Bt_i8, col_scale = _rows_quantize(B.T, sr, 1e-12, col_absmax=b_col_absmax)
    if transposed_out:
        return gn_kernels.scaled_mm_t(A_i8, Bt_i8.T, row_scale, col_scale.view(1, -1))
    return scaled_mm(A_i8, Bt_i8.T, row_scale, col_scale.view(1, -1))


def _dynamic_mm(A, B, sr, dtype, **kw):
    if dtype == "int8":
        return _dynamic_int8_mm(A, B, sr, **kw)
    if dtype == "int4":
        raise NotImplementedError("INT4 matmuls need int4 tensor cores, which B200 does not have")
    raise ValueError(dtype)


class _Int8MixedPrecisionLinear(torch.autograd.Function):
    """forward X W^T, grad_input dY W, grad_weight (X^T dY)^T, each optionally through INT8
    (reference: mixed_precision.py:146-193)."""

    @staticmethod
    def forward(input: Tensor, weight: MixedPrecisionLinearWeight, bias: Tensor | None = None):
        cfg = weight.config
        if cfg.output:
            batch_dims = input.shape[:-1]
            x2d = input.reshape(-1, weight.shape[1])
            # the same hidden state usually feeds several projections: quantize it once
            out = _dynamic_mm(x2d, weight._data.T, cfg.stochastic_rounding, cfg.dtype, cache_a=True)
            out = out.view(*batch_dims, weight.shape[0])
        else:
            out = input @ weight._data.T
        return out + bias if bias is not None else out

    @staticmethod
    def setup_context(ctx, inputs, output):
        input, weight, bias = inputs
        ctx.config = weight.config
        ctx.save_for_backward(input, weight._data)
        ctx.bias = bias is not None

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        cfg = ctx.config
        grad_input = grad_weight = grad_bias = None
        _quant_cache.clear_after_backward()   # cached activations must not outlive the step

        batch_dims = grad_output.shape[:-1]
        gy = grad_output.reshape(-1, weight.shape[0])
        x2d = input.reshape(-1, weight.shape[1])
        sr = cfg.stochastic_rounding

        gy_colmax = None
        if ctx.needs_input_grad[0]:
            if cfg.grad_input:
                if cfg.dtype == "int8" and cfg.grad_weight and ctx.needs_input_grad[1]:
                    # one pass over dY yields its row-wise int8 AND the column maxima that the
                    # grad-weight quantize of dY needs
                    gy_i8, gy_scale, gy_colmax = gn_kernels.quantize_rowwise_colabsmax(gy, torch.int8, sr)
                    wt_i8, w_colscale = _rows_quantize(weight.T, sr, 1e-12)
                    grad_input = scaled_mm(gy_i8, wt_i8.T, gy_scale, w_colscale.view(1, -1))
                else:
                    grad_input = _dynamic_mm(gy, weight, sr, cfg.dtype)
            else:
                grad_input = gy @ weight
            grad_input = grad_input.view(*batch_dims, weight.shape[1])

        if ctx.needs_input_grad[1]:
            if cfg.grad_weight:
                # a fused producer (gn_kernels.fused) may have left the activation's column maxima on the tensor
                x_colmax = getattr(input, "_qt_col_absmax", None) if cfg.dtype == "int8" else None
                # (X^T dY)^T written straight into the weight's [N, K] layout (a strided gradient would be copied again)
                grad_weight = _dynamic_mm(x2d.T, gy, sr, cfg.dtype, a_col_absmax=x_colmax, b_col_absmax=gy_colmax, cache_a=True,
                                          transposed_out=True)
            else:
                grad_weight = gy.T @ x2d

        if len(ctx.needs_input_grad) > 2 and ctx.needs_input_grad[2] and ctx.bias:
            grad_bias = gy.sum(0)

        return grad_input, grad_weight, grad_bias


def convert_mixed_precision(module: nn.Module, *, config: MixedPrecisionConfig = MixedPrecisionConfig()):
    """Wrap every nn.Linear weight under `module` (mixed_precision.py:196-205)."""
    if isinstance(module, nn.Linear):
        module.weight = nn.Parameter(
            MixedPrecisionLinearWeight(module.weight.detach(), config=config),
            requires_grad=module.weight.requires_grad,
        )
    else:
        for m in module.children():
            convert_mixed_precision(m, config=config)
    return module


# ---- the gathered form of the weight under FSDP2 ------------------------------------------------


class Int8RowScaledLinearWeight(Tensor):
    """Unsharded weight as it comes out of the INT8 all-gather: int8 rows [N,K] + scale [N,1].

    Forward uses the gathered int8 rows directly (no weight quantize). Backward keeps using the
    SAME quantized weight: grad_input = rowquant(dY * scale^T) @ W_i8 (the weight scale is folded
    into dY before its row-wise quantize, so W needs no column-wise re-quantize), and grad_weight
    is the dynamic INT8 matmul of the reference. Container only: it lives for one forward/backward.
    """

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, int_data: Tensor, scale: Tensor, config: MixedPrecisionConfig, mode: str = "row", col_scale: Tensor | None = None):
        return Tensor._make_wrapper_subclass(cls, int_data.shape, dtype=scale.dtype, device=int_data.device)

    @torch._dynamo.disable
    def __init__(self, int_data: Tensor, scale: Tensor, config: MixedPrecisionConfig, mode: str = "row", col_scale: Tensor | None = None):
        assert int_data.dtype is torch.int8 and int_data.ndim == 2
        self.int_data = int_data
        self.scale = scale
        self.config = config
        # "row": int_data rows carry `scale` (the forward gather). "col": int_data was quantized along the
        # output dimension with the [K, 1] `col_scale` (the backward gather) and `scale` is unused.
        self.mode = mode
        self.col_scale = col_scale

    def __tensor_flatten__(self):
        return ["int_data", "scale"], [self.config]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["int_data"], tensor_data_dict["scale"], *tensor_attributes)

    def __repr__(self):
        return f"{self.__class__.__name__}(shape={tuple(self.shape)}, config={self.config})"

    def dequantize(self):
        if self.mode == "col":
            return self.int_data * self.col_scale.view(1, -1)
        return self.int_data * self.scale.view(-1, 1)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or dict()
        if func is F.linear:
            return _Int8GatheredLinear.apply(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = kwargs or {}
        if func in (aten.detach.default, aten.clone.default):
            w = args[0]
            return cls(func(w.int_data, *args[1:], **kwargs), func(w.scale, *args[1:], **kwargs), w.config, w.mode, w.col_scale)
        if func is aten.as_strided.default:
            w = args[0]
            return cls(w.int_data, w.scale, w.config, w.mode, w.col_scale)
        raise NotImplementedError(f"{cls.__name__} dispatch: attempting to run {func}, this is not supported")


class _Int8GatheredLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: Tensor, weight: Int8RowScaledLinearWeight, bias: Tensor | None = None):
        cfg = weight.config
        if weight.mode != "row":
            raise RuntimeError(
                "the gathered INT8 weight holds the backward (column-wise) quantization but a forward product asked for it: with "
                "activation checkpointing the recomputed forward runs on the backward gather; set "
                "MixedPrecisionLinearWeight.backward_gather = 'row'")
        batch_dims = input.shape[:-1]
        x2d = input.reshape(-1, weight.shape[1])
        sr = cfg.stochastic_rounding
        x_i8, x_scale = _rows_quantize(x2d, sr, 1e-12, cache=True)
        out = scaled_mm(x_i8, weight.int_data.T, x_scale, weight.scale.view(1, -1))
        ctx.save_for_backward(input, weight.int_data, weight.scale)
        ctx.weight_obj = weight   # its mode / col_scale are read in backward, after FSDP2 may have gathered again
        ctx.config = cfg
        ctx.bias = bias is not None
        out = out.view(*batch_dims, weight.shape[0])
        return out + bias if bias is not None else out

    @staticmethod
    def backward(ctx, grad_output):
        input, w_i8, w_scale = ctx.saved_tensors
        cfg = ctx.config
        sr = cfg.stochastic_rounding
        grad_input = grad_weight = grad_bias = None
        batch_dims = grad_output.shape[:-1]
        gy = grad_output.reshape(-1, w_i8.shape[0])
        x2d = input.reshape(-1, w_i8.shape[1])

        _quant_cache.clear_after_backward()
        wobj = ctx.weight_obj
        gy_colmax = None
        if ctx.needs_input_grad[0]:
            if wobj.mode == "col":
                # the reference's grad-input product: rows of dY against the weight quantized along its
                # output dimension (subclasses/mixed_precision.py:176-178); w_i8 [N, K] is that quantization
                if cfg.grad_weight and ctx.needs_input_grad[1]:
                    g_i8, g_scale, gy_colmax = gn_kernels.quantize_rowwise_colabsmax(gy, torch.int8, sr)
                else:
                    g_i8, g_scale = gn_kernels.quantize_rowwise(gy, torch.int8, sr)
                grad_input = scaled_mm(g_i8, w_i8, g_scale, wobj.col_scale.view(1, -1))
            else:
                # only the forward's row-wise quantization is at hand: its row scales go into dY
                gy_scaled = gy * w_scale.view(1, -1)
                g_i8, g_scale = gn_kernels.quantize_rowwise(gy_scaled, torch.int8, sr)
                one = torch.ones((1, 1), dtype=g_scale.dtype, device=g_scale.device)
                grad_input = scaled_mm(g_i8, w_i8, g_scale, one)
            grad_input = grad_input.view(*batch_dims, w_i8.shape[1])

        if ctx.needs_input_grad[1]:
            if cfg.grad_weight:
                x_colmax = getattr(input, "_qt_col_absmax", None)
                grad_weight = _dynamic_int8_mm(x2d.T, gy, sr, a_col_absmax=x_colmax, b_col_absmax=gy_colmax, cache_a=True, transposed_out=True)
            else:
                grad_weight = gy.T @ x2d

        if len(ctx.needs_input_grad) > 2 and ctx.needs_input_grad[2] and ctx.bias:
            grad_bias = gy.sum(0)
        return grad_input, grad_weight, grad_bias
