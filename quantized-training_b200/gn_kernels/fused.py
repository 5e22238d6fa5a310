"""Producer-fused activation quantize and the other element-wise pieces of a decoder block.

`rmsnorm` and `silu_mul` are the two producers of the activations that feed INT8 linear layers in a
Llama-style block. Each runs as one kernel that writes the bf16 result and, on request, its row-wise
INT8 quantization plus per-column maxima from the same pass, so the linear layers that follow do not
read the activation again to quantize it (the optimisation the reference names at
subclasses/int8.py:155-156). `rope` is rotary position embedding in one pass. All three are autograd
functions with single-kernel backward passes.

How the quantized copy reaches its consumers: the (int8, scale) pair is parked in the activation cache
of `subclasses.int8` under the identity of the bf16 tensor, which the following linear layers look up
before they quantize; the column maxima (needed for the grad-weight quantize of the same activation in
backward) ride on the tensor object as `_qt_col_absmax`. A consumer that does not find them quantizes
as usual, with identical results.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _native as nv


def _rows2d(t: Tensor) -> Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < t2.shape[1]):
        t2 = t2.contiguous()
    return t2


def _stride0(t2: Tensor) -> int:
    return t2.stride(0) if t2.shape[0] > 1 else max(t2.shape[1], 1)


def _rows_per_cta(cols: int) -> int:
    return 8 if cols <= 1024 else (4 if cols <= 2048 else (2 if cols <= 4096 else 1))


def producer_supported(x: Tensor, cols: int | None = None) -> bool:
    """True when the fused producer kernels take this activation (bf16 on CUDA, last dimension a multiple
    of 8 and at most 16384, a row count the kernel's row grouping divides)."""
    if not (isinstance(x, Tensor) and x.is_cuda and x.dtype is torch.bfloat16 and x.ndim >= 2):
        return False
    cols = x.shape[-1] if cols is None else cols
    rows = x.numel() // max(cols, 1)
    return cols % 8 == 0 and 0 < cols <= 16384 and rows > 0 and rows % _rows_per_cta(cols) == 0


def _park_quantized(y: Tensor, q: Tensor, scale: Tensor, colmax: Tensor) -> None:
    from subclasses.int8 import _quant_cache

    y2 = y.view(-1, y.shape[-1])
    if _quant_cache.cacheable(y2) and not torch.compiler.is_compiling():
        _quant_cache.put(y2, 1e-12, (q, scale))
    y._qt_col_absmax = colmax


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, eps: float, emit_quant: bool):
        x2 = _rows2d(x)
        dev = nv.require_cuda(x2, weight)
        rows, cols = x2.shape
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=dev)
        rstd = torch.empty((rows,), dtype=torch.float32, device=dev)
        w = weight.detach().contiguous()
        q = scale = colmax = None
        if emit_quant:
            q = torch.empty((rows, cols), dtype=torch.int8, device=dev)
            scale = torch.empty((rows, 1), dtype=torch.bfloat16, device=dev)
            colmax = torch.empty((cols,), dtype=torch.float32, device=dev)
        with nv.on_device(dev):
            nv.check(nv.load().qt_rmsnorm_quantize(
                x2.data_ptr(), rows, cols, _stride0(x2), w.data_ptr(), float(eps), y.data_ptr(), rstd.data_ptr(),
                None if q is None else q.data_ptr(), nv.QT_I8, None if q is None else scale.data_ptr(), nv.QT_BF16,
                None if q is None else colmax.data_ptr(), 1e-12, nv.stream_ptr(dev)))
        ctx.save_for_backward(x2, w, rstd)
        ctx.x_shape = x.shape
        ctx.mark_non_differentiable(rstd)
        if emit_quant:
            _last_quant.append((q, scale, colmax))
        return y, rstd

    @staticmethod
    def backward(ctx, dy: Tensor, _drstd):
        x2, w, rstd = ctx.saved_tensors
        dev = x2.device
        rows, cols = x2.shape
        dy2 = _rows2d(dy)
        dx = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
        dw = torch.empty((cols,), dtype=w.dtype, device=dev)
        lib = nv.load()
        n_partial = lib.qt_rmsnorm_backward_partial_rows(rows, cols)
        partial = torch.empty((max(n_partial, 1), cols), dtype=torch.float32, device=dev)
        with nv.on_device(dev):
            nv.check(lib.qt_rmsnorm_backward(
                dy2.data_ptr(), _stride0(dy2), x2.data_ptr(), _stride0(x2), w.data_ptr(), rstd.data_ptr(), rows, cols,
                dx.data_ptr(), partial.data_ptr(), n_partial, dw.data_ptr(), nv.code(dw.dtype), nv.stream_ptr(dev)))
        return dx.view(ctx.x_shape), dw, None, None


def rmsnorm(x: Tensor, weight: Tensor, eps: float = 1e-6, *, emit_quant: bool = False) -> Tensor:
    """weight * bf16(x * rsqrt(mean(x^2) + eps)) over the last dimension (an eager RMSNorm module's
    arithmetic on bf16 input). With `emit_quant` the kernel also leaves the row-wise INT8 quantization
    of the result where the INT8 linear layers that consume it will find it."""
    y, _ = _RMSNorm.apply(x, weight, eps, emit_quant)
    if emit_quant:
        _park_quantized(y, *_last_quant.pop())
    return y


class _SiluMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: Tensor, up: Tensor, emit_quant: bool):
        g2, u2 = _rows2d(gate), _rows2d(up)
        dev = nv.require_cuda(g2, u2)
        rows, cols = g2.shape
        y = torch.empty(gate.shape, dtype=torch.bfloat16, device=dev)
        q = scale = colmax = None
        if emit_quant:
            q = torch.empty((rows, cols), dtype=torch.int8, device=dev)
            scale = torch.empty((rows, 1), dtype=torch.bfloat16, device=dev)
            colmax = torch.empty((cols,), dtype=torch.float32, device=dev)
        with nv.on_device(dev):
            nv.check(nv.load().qt_silu_mul_quantize(
                g2.data_ptr(), u2.data_ptr(), rows, cols, _stride0(g2), _stride0(u2), y.data_ptr(),
                None if q is None else q.data_ptr(), nv.QT_I8, None if q is None else scale.data_ptr(), nv.QT_BF16,
                None if q is None else colmax.data_ptr(), 1e-12, nv.stream_ptr(dev)))
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        if emit_quant:
            _last_quant.append((q, scale, colmax))
        return y

    @staticmethod
    def backward(ctx, dh: Tensor):
        g2, u2 = ctx.saved_tensors
        dev = g2.device
        rows, cols = g2.shape
        d2 = _rows2d(dh)
        dg = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
        du = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
        with nv.on_device(dev):
            nv.check(nv.load().qt_silu_mul_backward(
                d2.data_ptr(), _stride0(d2), g2.data_ptr(), _stride0(g2), u2.data_ptr(), _stride0(u2), rows, cols,
                dg.data_ptr(), du.data_ptr(), nv.stream_ptr(dev)))
        return dg.view(ctx.shape), du.view(ctx.shape), None


def silu_mul(gate: Tensor, up: Tensor, *, emit_quant: bool = False) -> Tensor:
    """bf16(bf16(silu(gate)) * up), the gated activation of a SwiGLU MLP, optionally leaving its row-wise
    INT8 quantization for the down projection."""
    y = _SiluMul.apply(gate, up, emit_quant)
    if emit_quant:
        _park_quantized(y, *_last_quant.pop())
    return y


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, cos: Tensor, sin: Tensor):
        # x: [batch, seq, heads, dim] contiguous; cos, sin: [batch or 1, seq, dim]
        ctx.save_for_backward(cos, sin)
        return _rope_call(x, cos, sin, 0)

    @staticmethod
    def backward(ctx, dy: Tensor):
        cos, sin = ctx.saved_tensors
        return _rope_call(dy.contiguous(), cos, sin, 1), None, None


def _rope_call(x: Tensor, cos: Tensor, sin: Tensor, inverse: int) -> Tensor:
    dev = nv.require_cuda(x, cos, sin)
    b, s, h, d = x.shape
    y = torch.empty_like(x)
    with nv.on_device(dev):
        nv.check(nv.load().qt_rope(x.data_ptr(), b * s, h, d, cos.data_ptr(), sin.data_ptr(), s,
                                   0 if cos.shape[0] == 1 else s * d, inverse, y.data_ptr(), nv.stream_ptr(dev)))
    return y


def rope_supported(x: Tensor, cos: Tensor, sin: Tensor) -> bool:
    return (x.is_cuda and x.dtype is torch.bfloat16 and x.ndim == 4 and x.is_contiguous() and x.shape[-1] % 16 == 0
            and cos.dtype is torch.bfloat16 and sin.dtype is torch.bfloat16 and cos.ndim == 3 and cos.shape == sin.shape
            and cos.is_contiguous() and sin.is_contiguous() and cos.shape[0] in (1, x.shape[0])
            and cos.shape[1] == x.shape[1] and cos.shape[2] == x.shape[3])


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotary position embedding of x [batch, seq, heads, dim] with cos / sin [batch or 1, seq, dim]:
    x * cos + rotate_half(x) * sin, one rounding per output."""
    return _Rope.apply(x, cos, sin)


# The forward of a producer leaves the quantized copy of its result here for the wrapper around apply() to
# pick up (the autograd context must not hold it: it would then live until backward).
_last_quant: list = []
