"""The debug library (-DQT_BOUNDS_CHECK on the quantize kernels) against the release library.

Every global store of the quantize kernels in that build first checks its address against the output ranges
the entry point declared, and a store outside them would be skipped and recorded in the device status word.
Here the two libraries run the same calls on ragged, strided and tiny shapes: the outputs must be identical,
byte for byte, and the status word must stay 0 -- i.e. no kernel ever tried to write outside its outputs.
Nothing in this file makes a kernel write out of bounds."""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

from gn_kernels import _native as nv  # noqa: E402

CHECK_LIB = Path(nv.__file__).resolve().parent / "libqt_b200_check.so"


@pytest.fixture(scope="module")
def libs():
    if not CHECK_LIB.exists():
        # normally built beside the release library; build it here (nvcc, a minute or two) when it is not
        import importlib.util

        spec = importlib.util.spec_from_file_location("qt_b200_build", CHECK_LIB.parents[1] / "csrc" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_checked()
    chk = ctypes.CDLL(str(CHECK_LIB))
    for name, (res, args) in nv.SIGNATURES.items():
        fn = getattr(chk, name)
        fn.restype, fn.argtypes = res, args
    return nv.load(), chk


def _status(lib):
    out = ctypes.c_int(-1)
    assert lib.qt_device_status(ctypes.byref(out)) == 0
    return out.value


SHAPES = [(1, 8), (3, 24), (9, 37), (50, 1001), (7, 520), (64, 1024), (129, 2048), (257, 1000), (33, 4104), (5, 16392), (2, 33000)]


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("stochastic", [0, 1])
def test_rowwise_and_column_maxima(libs, rows, cols, stochastic):
    rel, chk = libs
    dev = torch.device("cuda")
    stride = cols + (8 if cols % 8 == 0 else 3)
    x = (torch.randn(rows, stride, device=dev) * 3).bfloat16()[:, :cols]
    outs = []
    for lib in (rel, chk):
        q = torch.full((rows, cols), 77, dtype=torch.int8, device=dev)
        s = torch.zeros((rows, 1), dtype=torch.bfloat16, device=dev)
        cm = torch.zeros((cols,), dtype=torch.float32, device=dev)
        stream = nv.stream_ptr(dev)
        rc = lib.qt_quantize_rowwise(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), q.data_ptr(), nv.QT_I8, s.data_ptr(), nv.QT_BF16,
                                     1e-12, stochastic, 11, 5, stream)
        assert rc == 0, lib.qt_last_error()
        q2 = torch.full((rows, cols), 77, dtype=torch.int8, device=dev)
        s2 = torch.zeros((rows, 1), dtype=torch.bfloat16, device=dev)
        rc = lib.qt_quantize_rowwise_colabsmax(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), q2.data_ptr(), nv.QT_I8, s2.data_ptr(),
                                               nv.QT_BF16, cm.data_ptr(), 1e-12, stochastic, 11, 5, stream)
        assert rc == 0, lib.qt_last_error()
        torch.cuda.synchronize()
        outs.append((q, s, q2, s2, cm))
    assert _status(chk) == 0
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rows,cols", [(4, 8), (100, 72), (128, 64), (1000, 1536), (777, 520), (130, 4100)])
def test_columnwise_forms(libs, rows, cols):
    rel, chk = libs
    dev = torch.device("cuda")
    x = (torch.randn(rows, cols, device=dev) * 2).bfloat16()
    outs = []
    for lib in (rel, chk):
        stream = nv.stream_ptr(dev)
        cm = torch.zeros((cols,), dtype=torch.float32, device=dev)
        assert lib.qt_col_absmax(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), cm.data_ptr(), stream) == 0
        qt = torch.full((cols, rows), 55, dtype=torch.int8, device=dev)
        st = torch.zeros((cols, 1), dtype=torch.bfloat16, device=dev)
        rc = lib.qt_quantize_colwise_t(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), cm.data_ptr(), qt.data_ptr(), nv.QT_I8, st.data_ptr(),
                                       nv.QT_BF16, 1e-12, 0, 0, 0, stream)
        assert rc == 0, lib.qt_last_error()
        q = torch.full((rows, cols), 55, dtype=torch.int8, device=dev)
        s = torch.zeros((1, cols), dtype=torch.bfloat16, device=dev)
        rc = lib.qt_quantize_colwise(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), cm.data_ptr(), q.data_ptr(), nv.QT_I8, s.data_ptr(),
                                     nv.QT_BF16, 1e-12, 0, 0, 0, stream)
        assert rc == 0, lib.qt_last_error()
        torch.cuda.synchronize()
        outs.append((qt, st, q, s))
    assert _status(chk) == 0
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rows,cols,tile_r", [(5, 128, 1), (64, 1024, 1), (33, 2048, 1), (100, 200, 1), (128, 128, 128), (256, 1024, 128), (130, 300, 128)])
def test_tile_forms(libs, rows, cols, tile_r):
    rel, chk = libs
    dev = torch.device("cuda")
    x = torch.randn(rows, cols, device=dev).bfloat16()
    sr, sc = (rows + tile_r - 1) // tile_r, (cols + 127) // 128
    outs = []
    for lib in (rel, chk):
        q = torch.full((rows, cols), 33, dtype=torch.int8, device=dev)
        s = torch.zeros((sr, sc), dtype=torch.bfloat16, device=dev)
        rc = lib.qt_quantize_tile(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), tile_r, 128, q.data_ptr(), nv.QT_I8, s.data_ptr(), nv.QT_BF16,
                                  1e-12, nv.stream_ptr(dev))
        assert rc == 0, lib.qt_last_error()
        torch.cuda.synchronize()
        outs.append((q, s))
    assert _status(chk) == 0
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rows,cols", [(8, 64), (24, 1024), (96, 2048), (40, 5632)])
def test_producer_forms_and_weight_update(libs, rows, cols):
    rel, chk = libs
    dev = torch.device("cuda")
    x = torch.randn(rows, cols, device=dev).bfloat16()
    u = torch.randn(rows, cols, device=dev).bfloat16()
    w = torch.randn(cols, device=dev).bfloat16()
    outs = []
    for lib in (rel, chk):
        stream = nv.stream_ptr(dev)
        res = []
        for producer in ("rmsnorm", "silu"):
            y = torch.zeros((rows, cols), dtype=torch.bfloat16, device=dev)
            q = torch.full((rows, cols), 9, dtype=torch.int8, device=dev)
            s = torch.zeros((rows, 1), dtype=torch.bfloat16, device=dev)
            cm = torch.zeros((cols,), dtype=torch.float32, device=dev)
            if producer == "rmsnorm":
                rstd = torch.zeros((rows,), dtype=torch.float32, device=dev)
                rc = lib.qt_rmsnorm_quantize(x.data_ptr(), rows, cols, cols, w.data_ptr(), 1e-6, y.data_ptr(), rstd.data_ptr(), q.data_ptr(), nv.QT_I8,
                                             s.data_ptr(), nv.QT_BF16, cm.data_ptr(), 1e-12, stream)
                res.append(rstd)
            else:
                rc = lib.qt_silu_mul_quantize(x.data_ptr(), u.data_ptr(), rows, cols, cols, cols, y.data_ptr(), q.data_ptr(), nv.QT_I8, s.data_ptr(),
                                              nv.QT_BF16, cm.data_ptr(), 1e-12, stream)
            assert rc == 0, lib.qt_last_error()
            res += [y, q, s, cm]
        # the fused INT8 weight update on a copy of one quantized result
        qw, sw = res[2].clone(), res[3].clone()
        rc = lib.qt_int8_weight_update(qw.data_ptr(), sw.data_ptr(), rows, cols, 0, u.data_ptr(), None, -0.01, 1e-12, 3, 9, stream)
        assert rc == 0, lib.qt_last_error()
        torch.cuda.synchronize()
        outs.append(res + [qw, sw])
    assert _status(chk) == 0
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
