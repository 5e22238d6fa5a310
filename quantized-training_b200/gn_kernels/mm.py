"""int8_mm / scaled_mm / tile_scaled_mm with the reference's names, schemas and argument checks
(kernels/gn_kernels/triton_mm.py:112-128,345-441), running on the tcgen05 kernels."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _native as nv
from ._lib import lib, lib_ops

_F8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def _operand(t: Tensor, k_dim: int) -> Tensor:
    """Return `t` (or a re-laid-out copy) that the TMA path accepts: one unit stride, the other a
    multiple of 16 bytes, 16-byte aligned base. K-major copies are padded along K with zeros."""
    mn_dim = 1 - k_dim
    s_k, s_mn = t.stride(k_dim), t.stride(mn_dim)
    n_k, n_mn = t.shape[k_dim], t.shape[mn_dim]
    ok_kmajor = s_k == 1 and s_mn % 16 == 0 and s_mn >= n_k
    ok_mnmajor = s_mn == 1 and s_k % 16 == 0 and s_k >= n_mn
    if (ok_kmajor or ok_mnmajor) and t.data_ptr() % 16 == 0 and n_k > 1 and n_mn > 1:
        return t
    # rebuild as K-major with a padded pitch
    pitch = max(16, -(-n_k // 16) * 16)
    buf = torch.zeros((n_mn, pitch), dtype=t.dtype, device=t.device)
    view = buf[:, :n_k]
    view.copy_(t if k_dim == 1 else t.T)
    return view if k_dim == 1 else view.T


def _direct(*tensors: Tensor) -> bool:
    """Plain CUDA tensors outside torch.compile tracing: call the kernel without the dispatcher."""
    if torch.compiler.is_compiling():
        return False
    return all(type(t) is Tensor and t.is_cuda for t in tensors)


def _workspace(M: int, N: int, K: int, dev: torch.device):
    """(tensor or None, pointer, bytes) of the split-K scratch the library asks for; (None, 0, 0) for most
    shapes. Only small outputs with long reductions (M * N up to a few hundred tiles) ever split, so this is
    cheap. The caller holds the tensor until its launch is enqueued; after that the caching allocator may hand
    the block to later work of the same stream only, which runs after the kernel (no state is shared between
    the threads that call into this module)."""
    if M * N > (1 << 23) or K < 2048:
        return None, 0, 0
    need = nv.load().qt_gemm_workspace_bytes(M, N, K)
    if need <= 0:
        return None, 0, 0
    buf = torch.empty(need, dtype=torch.uint8, device=dev)
    return buf, buf.data_ptr(), need


lib.define("int8_mm(Tensor A, Tensor B) -> Tensor")
lib.define("scaled_mm(Tensor A, Tensor B, Tensor scale_A, Tensor scale_B) -> Tensor")
lib.define("tile_scaled_mm(Tensor A, Tensor B, Tensor scale_A, Tensor scale_B) -> Tensor")


def int8_mm(A: Tensor, B: Tensor) -> Tensor:
    """int32 C = A @ B for int8 A [M,K], B [K,N], any of the A@B.T / A@B / A.T@B layouts."""
    assert A.dtype is torch.int8 and B.dtype is torch.int8
    assert A.shape[1] == B.shape[0]
    return _int8_mm_cuda(A, B) if _direct(A, B) else lib_ops.int8_mm(A, B)


@torch.library.impl(lib, "int8_mm", "Meta")
def _(a: Tensor, b: Tensor):
    return torch.empty((a.shape[0], b.shape[1]), device=a.device, dtype=torch.int32)


@torch.library.impl(lib, "int8_mm", "CUDA")
def _int8_mm_cuda(A: Tensor, B: Tensor):
    dev = nv.require_cuda(A, B)
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty((M, N), dtype=torch.int32, device=dev)
    if M == 0 or N == 0:
        return C
    if K == 0:
        return C.zero_()
    A, B = _operand(A, 1), _operand(B, 0)
    with nv.on_device(dev):
        ws_buf, ws, ws_bytes = _workspace(M, N, K, dev)
        nv.check(nv.load().qt_int8_mm_ws(A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
                                         C.data_ptr(), C.stride(0), M, N, K, ws, ws_bytes, nv.stream_ptr(dev)))
        nv.raise_if_device_failed()
        del ws_buf
    return C


def scaled_mm(A: Tensor, B: Tensor, scale_A: Tensor, scale_B: Tensor) -> Tensor:
    """Matmul of quantized A [M,K] and B [K,N] (both int8 or both fp8) with de-scaling.

    Scale shapes select the variant, as in the reference wrapper (triton_mm.py:349-373):
      * `scale_A` [M,1] with `scale_B` [1,N] or [1,1]: row/column (or row/tensor) scaling;
      * otherwise tile-wise: `scale_A` [M/qm, K/qk], `scale_B` [K/qk, N/qn].
    Two conveniences the reference's own callers need but its wrapper rejects: `scale_B` given as
    [N,1] (Int8LinearWeight.scale, subclasses/int8.py:157) is read as [1,N], and a 0-dim `scale_B`
    (BitNet's tensor scale, subclasses/bitnet.py:140) as [1,1]. Output dtype = scale dtype.
    """
    assert (A.dtype == B.dtype == torch.int8) or (A.dtype in _F8 and B.dtype in _F8)
    assert scale_A.dtype == scale_B.dtype
    if scale_B.ndim == 0:
        scale_B = scale_B.view(1, 1)
    elif scale_B.ndim == 2 and scale_B.shape == (B.shape[1], 1) and B.shape[1] != 1 and scale_A.shape == (A.shape[0], 1):
        scale_B = scale_B.view(1, -1)
    assert A.ndim == B.ndim == scale_A.ndim == scale_B.ndim == 2
    assert A.shape[1] == B.shape[0]

    if scale_A.shape == (A.shape[0], 1) and scale_B.shape in ((1, B.shape[1]), (1, 1)):
        assert scale_A.is_contiguous()
        assert scale_B.is_contiguous()
        if _direct(A, B, scale_A, scale_B):
            return _scaled_mm_cuda(A, B, scale_A, scale_B)
        return lib_ops.scaled_mm(A, B, scale_A, scale_B)

    assert scale_A.shape[1] == scale_B.shape[0]
    if _direct(A, B, scale_A, scale_B):
        return _tile_scaled_mm_cuda(A, B, scale_A, scale_B)
    return lib_ops.tile_scaled_mm(A, B, scale_A, scale_B)


@torch.library.impl(lib, "scaled_mm", "Meta")
@torch.library.impl(lib, "tile_scaled_mm", "Meta")
def _(A: Tensor, B: Tensor, scale_A: Tensor, scale_B: Tensor):
    return torch.empty((A.shape[0], B.shape[1]), device=A.device, dtype=scale_A.dtype)


def _scale_dtype_ok(scale: Tensor) -> None:
    if scale.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"scales must be bfloat16 or float32, got {scale.dtype}")


def scaled_mm_t(A: Tensor, B: Tensor, scale_A: Tensor, scale_B: Tensor) -> Tensor:
    """(B^T @ A^T) written directly, rounding like (A @ B)^T: returns C^T [N, M] for A [M, K] with row scales
    `scale_A` [M, 1] and B [K, N] with column scales `scale_B` [1, N]. The epilogue multiplies by the scale
    of A first, as scaled_mm does, so the result is bit-identical to `scaled_mm(A, B, scale_A, scale_B).T`
    without the strided layout (used for grad-weight, which has to land in the weight's own layout)."""
    assert A.ndim == B.ndim == 2 and A.shape[1] == B.shape[0]
    assert scale_A.shape == (A.shape[0], 1) and scale_B.shape == (1, B.shape[1])
    if _direct(A, B, scale_A, scale_B):
        return _scaled_mm_cuda(B.T, A.T, scale_B.reshape(-1, 1), scale_A.reshape(1, -1), col_scale_first=True)
    return scaled_mm(A, B, scale_A, scale_B).T


@torch.library.impl(lib, "scaled_mm", "CUDA")
def _scaled_mm_cuda(A: Tensor, B: Tensor, row_scale: Tensor, col_scale: Tensor, col_scale_first: bool = False):
    dev = nv.require_cuda(A, B, row_scale, col_scale)
    _scale_dtype_ok(row_scale)
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty((M, N), dtype=row_scale.dtype, device=dev)
    if M == 0 or N == 0:
        return C
    if K == 0:
        return C.zero_()
    A, B = _operand(A, 1), _operand(B, 0)
    row_scale, col_scale = row_scale.contiguous(), col_scale.contiguous()
    with nv.on_device(dev):
        ws_buf, ws, ws_bytes = _workspace(M, N, K, dev)
        nv.check(nv.load().qt_scaled_mm_ws(
            A.data_ptr(), nv.code(A.dtype), A.stride(0), A.stride(1), B.data_ptr(), nv.code(B.dtype), B.stride(0),
            B.stride(1), row_scale.data_ptr(), col_scale.data_ptr(), int(col_scale.numel() == 1 and N != 1) | (2 if col_scale_first else 0),
            nv.code(row_scale.dtype), C.data_ptr(), C.stride(0), M, N, K, ws, ws_bytes, nv.stream_ptr(dev)))
        nv.raise_if_device_failed()
        del ws_buf
    return C


@torch.library.impl(lib, "tile_scaled_mm", "CUDA")
def _tile_scaled_mm_cuda(A: Tensor, B: Tensor, scale_A: Tensor, scale_B: Tensor):
    dev = nv.require_cuda(A, B, scale_A, scale_B)
    _scale_dtype_ok(scale_A)
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty((M, N), dtype=scale_A.dtype, device=dev)
    if M == 0 or N == 0:
        return C
    if K == 0:
        return C.zero_()
    qm, qk, qn = M // scale_A.shape[0], K // scale_A.shape[1], N // scale_B.shape[1]
    A, B = _operand(A, 1), _operand(B, 0)
    with nv.on_device(dev):
        nv.check(nv.load().qt_tile_scaled_mm(
            A.data_ptr(), nv.code(A.dtype), A.stride(0), A.stride(1), B.data_ptr(), nv.code(B.dtype), B.stride(0),
            B.stride(1), scale_A.data_ptr(), scale_A.stride(0), scale_A.stride(1), scale_B.data_ptr(), scale_B.stride(0),
            scale_B.stride(1), qm, qn, qk, nv.code(scale_A.dtype), C.data_ptr(), C.stride(0), M, N, K,
            nv.stream_ptr(dev)))
        nv.raise_if_device_failed()
    return C


def bf16_mm_colscale_supported(x2d: Tensor, w: Tensor, scale: Tensor) -> bool:
    return (x2d.is_cuda and x2d.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and scale.dtype is torch.bfloat16
            and x2d.ndim == 2 and w.ndim == 2 and x2d.shape[1] == w.shape[1] and scale.numel() == w.shape[0]
            and x2d.shape[1] % 8 == 0 and x2d.stride(1) == 1 and w.stride(1) == 1 and x2d.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x2d.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x2d.shape[0] > 0 and w.shape[0] > 0
            and not torch.compiler.is_compiling())


def bf16_mm_colscale(x2d: Tensor, w: Tensor, scale: Tensor) -> Tensor:
    """bf16(bf16(x2d @ w.T) * scale[None, :]) in one kernel: x2d [M, K], w [N, K], scale [N] (all bf16). The
    INT8 weight-only forward of the reference (subclasses/int8.py:147) with the per-channel multiply folded
    into the GEMM epilogue; both bf16 roundings of the two-step form are kept."""
    dev = nv.require_cuda(x2d, w, scale)
    M, K = x2d.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    scale = scale.reshape(-1).contiguous()
    with nv.on_device(dev):
        nv.check(nv.load().qt_bf16_mm_colscale(x2d.data_ptr(), x2d.stride(0), w.data_ptr(), w.stride(0), scale.data_ptr(), out.data_ptr(),
                                               N, M, N, K, nv.stream_ptr(dev)))
        nv.raise_if_device_failed()
    return out
