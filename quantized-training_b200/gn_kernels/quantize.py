"""Absmax quantize operators (row-wise, column-wise + transpose, tile-wise) on the sm_100a kernels.

The arithmetic is that of the reference's `quantize_int8` (subclasses/int8.py:12-26); these ops
exist so the quantize step is one HBM pass instead of a chain of eager / inductor kernels.
"""
from __future__ import annotations

import itertools
import threading

import torch
from torch import Tensor

from . import _native as nv
from ._lib import lib, lib_ops

_F8 = (torch.float8_e4m3fn, torch.float8_e5m2)
_philox_calls = itertools.count(1)
_philox_lock = threading.Lock()


def next_philox_key(device: torch.device) -> tuple[int, int]:
    """(seed, offset) for one stochastic-rounding launch: the seed follows torch.manual_seed on
    that device, the offset counts launches in this process, so runs are reproducible."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    seed = torch.cuda.default_generators[idx].initial_seed() & 0xFFFFFFFFFFFFFFFF
    with _philox_lock:
        return seed, next(_philox_calls)


def reserve_philox_keys(device: torch.device, n: int) -> tuple[int, int]:
    """(seed, first offset) of `n` consecutive launch offsets, for one call that stands for n launches."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    seed = torch.cuda.default_generators[idx].initial_seed() & 0xFFFFFFFFFFFFFFFF
    with _philox_lock:
        first = next(_philox_calls)
        for _ in range(n - 1):
            next(_philox_calls)
    return seed, first


def _rows_view(x: Tensor) -> Tensor:
    """2-D view with unit inner stride (copies only when the layout forces it)."""
    if x.ndim != 2:
        raise ValueError(f"expected a 2-D tensor, got shape {tuple(x.shape)}")
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"quantize kernels take bfloat16 or float32 input, got {x.dtype}")
    if x.shape[1] > 1 and x.stride(1) != 1:
        x = x.contiguous()
    if x.shape[0] > 1 and x.stride(0) < x.shape[1]:
        x = x.contiguous()
    return x


def _row_stride(x: Tensor) -> int:
    return x.stride(0) if x.shape[0] > 1 else max(x.shape[1], 1)


# Offset value that tells an op implementation to draw its (seed, offset) pair when it RUNS. Under
# torch.compile the Python wrapper is traced (by dynamo, or executed on fake / functional tensors by the later
# stages), and a pair drawn at trace time would be baked into the graph as constants: every step would then
# round with the same noise. The sentinel is what gets baked instead.
_DRAW_AT_RUN_TIME = -1


def _resolve_key(dev: torch.device, stochastic: bool, seed: int, offset: int) -> tuple[int, int]:
    if stochastic and offset == _DRAW_AT_RUN_TIME:
        return next_philox_key(dev)
    return seed, offset


# ---- op definitions ---------------------------------------------------------------------------

lib.define("quantize_rowwise(Tensor x, ScalarType out_dtype, ScalarType scale_dtype, bool stochastic, float eps, int seed, int offset) -> (Tensor, Tensor)")
lib.define("quantize_rowwise_colabsmax(Tensor x, ScalarType out_dtype, ScalarType scale_dtype, bool stochastic, float eps, int seed, int offset) -> (Tensor, Tensor, Tensor)")
lib.define("col_absmax(Tensor x) -> Tensor")
lib.define("quantize_colwise_t(Tensor x, Tensor col_absmax, ScalarType out_dtype, ScalarType scale_dtype, bool stochastic, float eps, int seed, int offset) -> (Tensor, Tensor)")
lib.define("quantize_tile(Tensor x, int tile_r, int tile_c, ScalarType out_dtype, ScalarType scale_dtype, float eps) -> (Tensor, Tensor)")


@torch.library.impl(lib, "quantize_rowwise", "Meta")
def _(x, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    return x.new_empty(x.shape, dtype=out_dtype), x.new_empty((x.shape[0], 1), dtype=scale_dtype)


@torch.library.impl(lib, "quantize_rowwise", "CUDA")
def _rowwise_cuda(x, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    x = _rows_view(x)
    dev = nv.require_cuda(x)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=out_dtype, device=dev)
    scale = torch.empty((rows, 1), dtype=scale_dtype, device=dev)
    seed, offset = _resolve_key(dev, stochastic, seed, offset)
    with nv.on_device(dev):
        nv.check(nv.load().qt_quantize_rowwise(
            x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x), q.data_ptr(), nv.code(out_dtype),
            scale.data_ptr(), nv.code(scale_dtype), eps, int(stochastic), seed, offset, nv.stream_ptr(dev)))
    return q, scale


@torch.library.impl(lib, "quantize_rowwise_colabsmax", "Meta")
def _(x, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    return (x.new_empty(x.shape, dtype=out_dtype), x.new_empty((x.shape[0], 1), dtype=scale_dtype),
            x.new_empty((x.shape[1],), dtype=torch.float32))


@torch.library.impl(lib, "quantize_rowwise_colabsmax", "CUDA")
def _rowwise_colabsmax_cuda(x, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    x = _rows_view(x)
    dev = nv.require_cuda(x)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=out_dtype, device=dev)
    scale = torch.empty((rows, 1), dtype=scale_dtype, device=dev)
    colmax = torch.empty((cols,), dtype=torch.float32, device=dev)
    seed, offset = _resolve_key(dev, stochastic, seed, offset)
    with nv.on_device(dev):
        nv.check(nv.load().qt_quantize_rowwise_colabsmax(
            x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x), q.data_ptr(), nv.code(out_dtype),
            scale.data_ptr(), nv.code(scale_dtype), colmax.data_ptr(), eps, int(stochastic), seed, offset,
            nv.stream_ptr(dev)))
    return q, scale, colmax


@torch.library.impl(lib, "col_absmax", "Meta")
def _(x):
    return x.new_empty((x.shape[1],), dtype=torch.float32)


@torch.library.impl(lib, "col_absmax", "CUDA")
def _col_absmax_cuda(x):
    x = _rows_view(x)
    dev = nv.require_cuda(x)
    rows, cols = x.shape
    colmax = torch.empty((cols,), dtype=torch.float32, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_col_absmax(x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x),
                                         colmax.data_ptr(), nv.stream_ptr(dev)))
    return colmax


@torch.library.impl(lib, "quantize_colwise_t", "Meta")
def _(x, col_absmax, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    return x.new_empty((x.shape[1], x.shape[0]), dtype=out_dtype), x.new_empty((x.shape[1], 1), dtype=scale_dtype)


@torch.library.impl(lib, "quantize_colwise_t", "CUDA")
def _colwise_t_cuda(x, col_absmax, out_dtype, scale_dtype, stochastic, eps, seed, offset):
    x = _rows_view(x)
    dev = nv.require_cuda(x, col_absmax)
    rows, cols = x.shape
    if col_absmax.dtype != torch.float32 or col_absmax.numel() != cols or not col_absmax.is_contiguous():
        raise ValueError("col_absmax must be a contiguous float32 tensor with one entry per column of x")
    qt = torch.empty((cols, rows), dtype=out_dtype, device=dev)
    scale = torch.empty((cols, 1), dtype=scale_dtype, device=dev)
    seed, offset = _resolve_key(dev, stochastic, seed, offset)
    with nv.on_device(dev):
        nv.check(nv.load().qt_quantize_colwise_t(
            x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x), col_absmax.data_ptr(), qt.data_ptr(),
            nv.code(out_dtype), scale.data_ptr(), nv.code(scale_dtype), eps, int(stochastic), seed, offset,
            nv.stream_ptr(dev)))
    return qt, scale


@torch.library.impl(lib, "quantize_tile", "Meta")
def _(x, tile_r, tile_c, out_dtype, scale_dtype, eps):
    sr, sc = -(-x.shape[0] // tile_r), -(-x.shape[1] // tile_c)
    return x.new_empty(x.shape, dtype=out_dtype), x.new_empty((sr, sc), dtype=scale_dtype)


@torch.library.impl(lib, "quantize_tile", "CUDA")
def _tile_cuda(x, tile_r, tile_c, out_dtype, scale_dtype, eps):
    x = _rows_view(x)
    dev = nv.require_cuda(x)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=out_dtype, device=dev)
    scale = torch.empty((-(-rows // tile_r), -(-cols // tile_c)), dtype=scale_dtype, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_quantize_tile(
            x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x), tile_r, tile_c, q.data_ptr(),
            nv.code(out_dtype), scale.data_ptr(), nv.code(scale_dtype), eps, nv.stream_ptr(dev)))
    return q, scale


# ---- Python wrappers --------------------------------------------------------------------------

def _key(x: Tensor, stochastic: bool) -> tuple[int, int]:
    if not stochastic:
        return 0, 0
    if torch.compiler.is_compiling() or type(x) is not Tensor:
        return 0, _DRAW_AT_RUN_TIME
    return next_philox_key(x.device)


def _direct(x: Tensor) -> bool:
    """True when the kernel can be called without going through the dispatcher: a plain CUDA tensor
    outside torch.compile tracing. The dispatcher round trip into a Python kernel costs about as much
    host time as the launch itself."""
    return type(x) is Tensor and x.is_cuda and not torch.compiler.is_compiling()


def quantize_rowwise(x: Tensor, out_dtype: torch.dtype = torch.int8, stochastic_rounding: bool = False, *,
                     eps: float = 1e-12, scale_dtype: torch.dtype | None = None, key: tuple[int, int] | None = None):
    """Per-row absmax quantize of a 2-D tensor: returns (q [R,C], scale [R,1]).

    `scale` comes back in `x.dtype` unless `scale_dtype` says otherwise, as quantize_int8 does
    (subclasses/int8.py:26). `key` = (seed, offset) pins the stochastic-rounding stream.
    """
    seed, offset = key if key is not None else _key(x, stochastic_rounding)
    fn = _rowwise_cuda if _direct(x) else lib_ops.quantize_rowwise
    return fn(x, out_dtype, scale_dtype or x.dtype, stochastic_rounding, eps, seed, offset)


def quantize_rowwise_colabsmax(x: Tensor, out_dtype: torch.dtype = torch.int8, stochastic_rounding: bool = False, *,
                               eps: float = 1e-12, scale_dtype: torch.dtype | None = None,
                               key: tuple[int, int] | None = None):
    """quantize_rowwise plus the per-column |x| maximum ([C] float32) from the same pass over x."""
    seed, offset = key if key is not None else _key(x, stochastic_rounding)
    fn = _rowwise_colabsmax_cuda if _direct(x) else lib_ops.quantize_rowwise_colabsmax
    return fn(x, out_dtype, scale_dtype or x.dtype, stochastic_rounding, eps, seed, offset)


def col_absmax(x: Tensor) -> Tensor:
    """Per-column |x| maximum of a 2-D tensor, float32 [C]."""
    return _col_absmax_cuda(x) if _direct(x) else lib_ops.col_absmax(x)


def quantize_colwise_t(x: Tensor, out_dtype: torch.dtype = torch.int8, stochastic_rounding: bool = False, *,
                       eps: float = 1e-12, scale_dtype: torch.dtype | None = None, col_absmax_: Tensor | None = None,
                       key: tuple[int, int] | None = None):
    """Per-column absmax quantize with the transpose materialised: returns (q [C,R], scale [C,1]),
    equal to quantizing `x.T` row-wise and calling `.contiguous()` (subclasses/mixed_precision.py:102-105)."""
    if col_absmax_ is None:
        col_absmax_ = col_absmax(x)
    seed, offset = key if key is not None else _key(x, stochastic_rounding)
    fn = _colwise_t_cuda if _direct(x) else lib_ops.quantize_colwise_t
    return fn(x, col_absmax_, out_dtype, scale_dtype or x.dtype, stochastic_rounding, eps, seed, offset)


def quantize_colwise(x: Tensor, col_absmax_: Tensor, out_dtype: torch.dtype = torch.int8, stochastic_rounding: bool = False, *,
                     eps: float = 1e-12, scale_dtype: torch.dtype | None = None, key: tuple[int, int] | None = None):
    """Per-column absmax quantize WITHOUT the transpose, from given column maxima: returns (q [R,C],
    scale [C,1]). For a row shard of a weight whose column maxima were agreed across the ranks."""
    x = _rows_view(x)
    dev = nv.require_cuda(x, col_absmax_)
    rows, cols = x.shape
    if col_absmax_.dtype != torch.float32 or col_absmax_.numel() != cols or not col_absmax_.is_contiguous():
        raise ValueError("col_absmax must be a contiguous float32 tensor with one entry per column of x")
    seed, offset = key if key is not None else (next_philox_key(dev) if stochastic_rounding else (0, 0))
    q = torch.empty((rows, cols), dtype=out_dtype, device=dev)
    scale = torch.empty((cols, 1), dtype=scale_dtype or x.dtype, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_quantize_colwise(
            x.data_ptr(), nv.code(x.dtype), rows, cols, _row_stride(x), col_absmax_.data_ptr(), q.data_ptr(), nv.code(out_dtype),
            scale.data_ptr(), nv.code(scale.dtype), eps, int(stochastic_rounding), seed, offset, nv.stream_ptr(dev)))
    return q, scale


def quantize_tile(x: Tensor, tile_shape: tuple[int, int], out_dtype: torch.dtype = torch.int8, *, eps: float = 1e-12,
                  scale_dtype: torch.dtype | None = None):
    """Per-tile absmax quantize (tiles 1x128 or 128x128): returns (q [R,C], scale [R/tr, C/tc])."""
    fn = _tile_cuda if _direct(x) else lib_ops.quantize_tile
    return fn(x, tile_shape[0], tile_shape[1], out_dtype, scale_dtype or x.dtype, eps)


def int8_weight_update_supported(int_data: Tensor, scale: Tensor, *operands: Tensor) -> bool:
    """True when the fused in-place update kernel takes these tensors (otherwise the caller
    de-quantizes, updates and re-quantizes in three steps)."""
    if not (int_data.is_cuda and int_data.dtype is torch.int8 and int_data.ndim == 2 and int_data.is_contiguous()):
        return False
    rows, cols = int_data.shape
    if cols % 8 != 0 or cols > 32768 or int_data.data_ptr() % 8:
        return False
    if scale.dtype is not torch.bfloat16 or scale.numel() != rows or not scale.is_contiguous() or scale.device != int_data.device:
        return False
    for t in operands:
        if not (isinstance(t, Tensor) and type(t) is Tensor and t.dtype is torch.bfloat16 and t.shape == int_data.shape
                and t.is_contiguous() and t.device == int_data.device and t.data_ptr() % 16 == 0):
            return False
    return True


def int8_weight_update_(int_data: Tensor, scale: Tensor, t1: Tensor, t2: Tensor | None, value: float, *,
                        eps: float = 1e-12, key: tuple[int, int] | None = None) -> None:
    """int_data, scale <- stochastic row-wise INT8 quantization of (int_data * scale) + value * t1
    (t2 is None) or + value * t1 / t2, in one pass and in place (reference: the de-quantize -> op ->
    re-quantize -> copy_ sequence of subclasses/int8.py:114-133)."""
    dev = nv.require_cuda(int_data, scale, t1, *(() if t2 is None else (t2,)))
    seed, offset = key if key is not None else next_philox_key(dev)
    rows, cols = int_data.shape
    with nv.on_device(dev):
        nv.check(nv.load().qt_int8_weight_update(
            int_data.data_ptr(), scale.data_ptr(), rows, cols, 0 if t2 is None else 1, t1.data_ptr(),
            None if t2 is None else t2.data_ptr(), float(value), float(eps), seed, offset, nv.stream_ptr(dev)))
