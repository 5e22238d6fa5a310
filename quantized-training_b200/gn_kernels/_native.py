"""ctypes binding of libqt_b200.so (the C ABI declared in include/qt_b200.h).

The library is the only compute path: if it is missing or a call fails this module raises,
it never falls back to PyTorch or CPU code.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).with_name("libqt_b200.so")

# element type codes of include/qt_b200.h
QT_BF16, QT_F32, QT_I8, QT_E4M3, QT_E5M2, QT_I32, QT_F16 = range(7)

DTYPE_CODE = {
    torch.bfloat16: QT_BF16,
    torch.float32: QT_F32,
    torch.int8: QT_I8,
    torch.float8_e4m3fn: QT_E4M3,
    torch.float8_e5m2: QT_E5M2,
    torch.int32: QT_I32,
    torch.float16: QT_F16,
}

# name -> (restype, argtypes): one entry per symbol of include/qt_b200.h
SIGNATURES = {
    "qt_last_error": (c_char_p, []),
    "qt_version": (c_char_p, []),
    "qt_device_status": (c_int, [ctypes.POINTER(c_int)]),
    "qt_device_status_peek": (c_int, [ctypes.POINTER(c_int)]),
    "qt_quantize_rowwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int,
                                    c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_quantize_rowwise_colabsmax": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p,
                                              c_int, c_void_p, c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_col_absmax": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "qt_quantize_colwise_t": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                                      c_int, c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_quantize_colwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                                    c_int, c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_quantize_colwise_t_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int,
                                              c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_quantize_tile": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int, c_void_p,
                                 c_int, c_float, c_void_p]),
    "qt_set_gemm_cta_group": (c_int, [c_int]),
    "qt_set_gemm_sm_margin": (c_int, [c_int]),
    "qt_set_gemm_group_m": (c_int, [c_int]),
    "qt_int8_mm": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                           c_int64, c_void_p]),
    "qt_scaled_mm": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p,
                             c_int, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "qt_bf16_mm_colscale": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "qt_gemm_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "qt_int8_mm_ws": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                              c_int64, c_void_p, c_int64, c_void_p]),
    "qt_scaled_mm_ws": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                c_int, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "qt_tile_scaled_mm": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64,
                                  c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                  c_int64, c_int64, c_int64, c_void_p]),
    "qt_abs_mean": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "qt_bitnet_quantize_weight": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_float, c_void_p, c_int, c_void_p]),
    "qt_unpack_i2": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "qt_adamw_bf16_sr": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_float, ctypes.c_double,
                                 ctypes.c_double, c_float, c_float, c_float, c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_quantize_rowwise_scatter": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, ctypes.POINTER(c_void_p),
                                            ctypes.POINTER(c_void_p), c_int64, c_int, c_int, c_float, c_void_p]),
    "qt_int8_weight_update": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_float, c_float,
                                      c_uint64, c_uint64, c_void_p]),
    "qt_adamw_bf16_sr_multi": (c_int, [c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                       ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), c_int, c_int, c_float, ctypes.c_double,
                                       ctypes.c_double, c_float, c_float, c_float, c_float, c_int, c_uint64, c_uint64, c_void_p]),
    "qt_rmsnorm_quantize": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int,
                                    c_void_p, c_int, c_void_p, c_float, c_void_p]),
    "qt_rmsnorm_backward_partial_rows": (c_int64, [c_int64, c_int64]),
    "qt_rmsnorm_backward": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                    c_int64, c_void_p, c_int, c_void_p]),
    "qt_silu_mul_quantize": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                                     c_int, c_void_p, c_float, c_void_p]),
    "qt_silu_mul_backward": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                     c_void_p]),
    "qt_rope": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "qt_selftest_wait_timeout": (c_int, [ctypes.POINTER(c_int), c_int]),
    "qt_selftest_division": (c_int, [c_int, c_float, ctypes.POINTER(ctypes.c_ulonglong)]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIB_PATH.exists():
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python quantized-training_b200/csrc/build.py` "
                        "(there is no fallback path)"
                    )
                lib = ctypes.CDLL(str(LIB_PATH))
                for name, (res, args) in SIGNATURES.items():
                    if not hasattr(lib, name):
                        continue  # optional symbols are checked by the tests against the header
                    fn = getattr(lib, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = lib
    return _lib


def check(rc: int) -> None:
    """Turn a non-zero return code into a RuntimeError carrying the library's message."""
    if rc != 0:
        msg = load().qt_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"qt_b200 error {rc}: {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """cudaStream_t of torch's current stream on `device` (the raw-handle query skips building a
    torch.cuda.Stream object: this is on the path of every kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def on_device(device: torch.device):
    """Context manager that makes `device` current for the C call; free when it already is."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} does not cross the qt_b200 boundary") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("qt_b200 kernels run on CUDA tensors only (there is no CPU path)")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


def device_status() -> int:
    """Status word written by kernels whose bounded waits ran out (0 = fine). Synchronises."""
    out = c_int(0)
    check(load().qt_device_status(ctypes.byref(out)))
    return out.value


_peek = c_int(0)


def raise_if_device_failed() -> None:
    """Raise RuntimeError when an earlier GEMM on the current device gave up on a bounded wait (its output
    is garbage). Reads a pinned host word the kernels write, so it costs no synchronisation; called after
    every GEMM launch, which means the error surfaces at the first launch after the failing kernel ran."""
    load().qt_device_status_peek(ctypes.byref(_peek))
    if _peek.value != 0:
        code = device_status()   # synchronises and clears
        raise RuntimeError(
            f"qt_b200: a GEMM kernel gave up on a bounded wait (status {code or _peek.value:#x}: role << 8 | barrier); "
            "results produced since the previous check are not valid")
