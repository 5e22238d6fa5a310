"""CPU checks of the boundary: the shared library loads and exports every symbol that
include/qt_b200.h declares, with a ctypes signature on the Python side; argument errors are
reported through return codes without touching a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "qt_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(qt_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as entry

    entry.build()
    from gn_kernels import _native

    return _native.load()


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("qt_quantize_rowwise", "qt_quantize_colwise_t", "qt_int8_mm", "qt_scaled_mm", "qt_tile_scaled_mm",
                 "qt_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from gn_kernels import _native

    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in qt_b200.h but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_native.SIGNATURES) <= set(declared_symbols())


def test_debug_library_with_store_guards_exports_the_same_symbols(lib):
    """build() also makes the -DQT_BOUNDS_CHECK library that the GPU store-guard test runs beside this one."""
    from gn_kernels import _native

    path = Path(_native.__file__).resolve().parent / "libqt_b200_check.so"
    assert path.exists(), "build() did not produce the debug library"
    chk = ctypes.CDLL(str(path))
    for name in declared_symbols():
        assert hasattr(chk, name), f"{name} missing from the debug library"


def test_version_and_error_strings(lib):
    assert b"sm_100a" in lib.qt_version()
    assert isinstance(lib.qt_last_error(), bytes)


def test_argument_errors_do_not_need_a_gpu(lib):
    # bad dtype code
    rc = lib.qt_quantize_rowwise(None, 99, 4, 4, 4, None, 2, None, 0, 1e-12, 0, 0, 0, None)
    assert rc == 1 and b"x_dtype" in lib.qt_last_error()
    # stride smaller than cols
    rc = lib.qt_quantize_rowwise(None, 0, 4, 8, 4, None, 2, None, 0, 1e-12, 0, 0, 0, None)
    assert rc == 1 and b"stride" in lib.qt_last_error()
    # GEMM: mixed operand families
    rc = lib.qt_scaled_mm(None, 2, 16, 1, None, 3, 1, 16, None, None, 0, 0, None, 16, 16, 16, 16, None)
    assert rc == 1
    # GEMM: misaligned pitch
    buf = ctypes.create_string_buffer(4096)
    addr = (ctypes.addressof(buf) + 15) & ~15
    rc = lib.qt_int8_mm(addr, 20, 1, addr, 1, 20, addr, 24, 24, 24, 20, None)
    assert rc == 1 and b"multiples of 16" in lib.qt_last_error()
    # unsupported tile shape
    rc = lib.qt_quantize_tile(addr, 0, 4, 4, 4, 3, 5, addr, 2, addr, 0, 1e-12, None)
    assert rc == 3
    # scatter form: destination count out of range, then a shape its kernel does not take
    ptrs = (ctypes.c_void_p * 1)(addr)
    rc = lib.qt_quantize_rowwise_scatter(addr, 0, 4, 8, 8, 0, ptrs, ptrs, 0, 2, 0, 1e-12, None)
    assert rc == 1 and b"destinations" in lib.qt_last_error()
    rc = lib.qt_quantize_rowwise_scatter(addr, 0, 4, 12, 16, 1, ptrs, ptrs, 0, 2, 0, 1e-12, None)
    assert rc == 3
    # optimizer and weight update: dtype and mode checks come before any launch
    rc = lib.qt_adamw_bf16_sr_multi(1, ptrs, ptrs, ptrs, ptrs, (ctypes.c_int64 * 1)(4), 2, 0, 1e-3, 0.9, 0.99, 0.0, 1e-8, 1.0, 1.0, 0, 0, 0, None)
    assert rc == 1 and b"dtype" in lib.qt_last_error()
    rc = lib.qt_int8_weight_update(addr, addr, 4, 8, 7, addr, addr, 1.0, 1e-12, 0, 0, None)
    assert rc == 1 and b"mode" in lib.qt_last_error()


def test_producer_and_gather_entry_points_check_their_arguments_on_the_host(lib):
    buf = ctypes.create_string_buffer(4096)
    addr = (ctypes.addressof(buf) + 15) & ~15
    # producers: bad quantized dtype; q without scale; a width the kernel does not take
    rc = lib.qt_rmsnorm_quantize(addr, 8, 64, 64, addr, 1e-6, addr, None, addr, 0, addr, 0, addr, 1e-12, None)
    assert rc == 1 and b"q_dtype" in lib.qt_last_error()
    rc = lib.qt_silu_mul_quantize(addr, addr, 8, 64, 64, 64, addr, addr, 2, None, 0, None, 1e-12, None)
    assert rc == 1 and b"without scale" in lib.qt_last_error()
    rc = lib.qt_rmsnorm_quantize(addr, 8, 60, 64, addr, 1e-6, addr, None, None, 2, None, 0, None, 1e-12, None)
    assert rc == 3 and b"multiple of 8" in lib.qt_last_error()
    # backward: scratch too small is an argument error, before any launch
    assert lib.qt_rmsnorm_backward_partial_rows(0, 64) == 0
    rc = lib.qt_rmsnorm_backward(addr, 64, addr, 64, addr, addr, 8, 64, addr, addr, 0, addr, 0, None)
    assert rc == 1 and b"dw_partial" in lib.qt_last_error()
    rc = lib.qt_silu_mul_backward(addr, 64, addr, 64, addr, 32, 8, 64, addr, addr, None)
    assert rc == 1 and b"stride" in lib.qt_last_error()
    # rotary embedding: tokens must be whole sequences; head size a multiple of 16
    rc = lib.qt_rope(addr, 10, 2, 64, addr, addr, 4, 0, 0, addr, None)
    assert rc == 1 and b"sequences" in lib.qt_last_error()
    rc = lib.qt_rope(addr, 8, 2, 24, addr, addr, 4, 0, 0, addr, None)
    assert rc == 3
    # bf16 GEMM with the scale in its epilogue: 16-byte rows
    rc = lib.qt_bf16_mm_colscale(addr, 20, addr, 20, addr, addr, 16, 16, 16, 20, None)
    assert rc == 3 and b"multiples of 8" in lib.qt_last_error()
    # scaled_mm flag bits beyond the two that are defined
    rc = lib.qt_scaled_mm(addr, 2, 16, 1, addr, 2, 1, 16, addr, addr, 4, 0, addr, 16, 16, 16, 16, None)
    assert rc == 1 and b"flag bits" in lib.qt_last_error()
    # column-wise quantize without the transpose: stochastic rounding is int8 only
    rc = lib.qt_quantize_colwise(addr, 0, 4, 8, 8, addr, addr, 3, addr, 0, 1e-12, 1, 0, 0, None)
    assert rc == 1 and b"stochastic" in lib.qt_last_error()


def test_python_ops_refuse_cpu_tensors():
    import torch
    import gn_kernels

    a = torch.zeros(16, 16, dtype=torch.int8)
    with pytest.raises((RuntimeError, NotImplementedError)):
        gn_kernels.int8_mm(a, a)
    with pytest.raises((RuntimeError, NotImplementedError)):
        gn_kernels.quantize_rowwise(torch.zeros(4, 8, dtype=torch.bfloat16))
