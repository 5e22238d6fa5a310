"""The allocation-free column-wise quantize (qt_quantize_colwise_t_noalloc), called through the C ABI.

Some hosts cannot let this library allocate: they own all device memory themselves (a server or
trainer with its own pool) or call from a place where allocation is not allowed. For them the
library keeps the per-column absmax scratch in a fixed array of its own. This test calls that entry
point twice in a row, on different inputs, and demands the same bytes and scales as the existing
two-call form (qt_col_absmax + qt_quantize_colwise_t with a caller buffer). The file name sorts
last on purpose, so a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from gn_kernels import _native as nv  # noqa: E402


def _two_call_form(x, stochastic=0, key=(0, 0)):
    rows, cols = x.shape
    colmax = torch.empty(cols, dtype=torch.float32, device=x.device)
    qt = torch.empty((cols, rows), dtype=torch.int8, device=x.device)
    scale = torch.empty((cols, 1), dtype=torch.bfloat16, device=x.device)
    lib, stream = nv.load(), nv.stream_ptr(x.device)
    nv.check(lib.qt_col_absmax(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), colmax.data_ptr(), stream))
    nv.check(lib.qt_quantize_colwise_t(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), colmax.data_ptr(), qt.data_ptr(),
                                       nv.QT_I8, scale.data_ptr(), nv.QT_BF16, 1e-12, stochastic, key[0], key[1], stream))
    return qt, scale


def _no_alloc_form(x, stochastic=0, key=(0, 0)):
    rows, cols = x.shape
    qt = torch.empty((cols, rows), dtype=torch.int8, device=x.device)
    scale = torch.empty((cols, 1), dtype=torch.bfloat16, device=x.device)
    nv.check(nv.load().qt_quantize_colwise_t_noalloc(x.data_ptr(), nv.QT_BF16, rows, cols, x.stride(0), qt.data_ptr(),
                                                     nv.QT_I8, scale.data_ptr(), nv.QT_BF16, 1e-12, stochastic, key[0],
                                                     key[1], nv.stream_ptr(x.device)))
    return qt, scale


def test_no_alloc_matches_two_call_form_on_two_calls_in_a_row():
    g = torch.Generator().manual_seed(123)
    # second input is smaller in magnitude and narrower: stale maxima from the first call would show
    first = (torch.randn(1000, 1536, generator=g) * 3.0).bfloat16().cuda()
    second = (torch.randn(777, 520, generator=g) * 0.01).bfloat16().cuda()
    for x in (first, second):
        want_q, want_s = _two_call_form(x)
        got_q, got_s = _no_alloc_form(x)
        torch.cuda.synchronize()
        assert torch.equal(got_q, want_q)
        assert torch.equal(got_s, want_s)
    # stochastic rounding takes the same route
    want_q, _ = _two_call_form(first, 1, (99, 7))
    got_q, _ = _no_alloc_form(first, 1, (99, 7))
    assert torch.equal(got_q, want_q)


def test_no_alloc_rejects_more_columns_than_its_scratch_holds():
    x = torch.zeros((1, 65536 + 8), dtype=torch.bfloat16, device="cuda")
    qt = torch.empty((65536 + 8, 1), dtype=torch.int8, device="cuda")
    scale = torch.empty((65536 + 8, 1), dtype=torch.bfloat16, device="cuda")
    rc = nv.load().qt_quantize_colwise_t_noalloc(x.data_ptr(), nv.QT_BF16, 1, 65536 + 8, 65536 + 8, qt.data_ptr(), nv.QT_I8,
                                                 scale.data_ptr(), nv.QT_BF16, 1e-12, 0, 0, 0, nv.stream_ptr(x.device))
    assert rc == 3
    assert b"65536" in nv.load().qt_last_error()
    # the limit itself is accepted
    x = torch.randn((4, 65536), device="cuda").bfloat16()
    got_q, got_s = _no_alloc_form(x)
    want_q, want_s = _two_call_form(x)
    assert torch.equal(got_q, want_q) and torch.equal(got_s, want_s)


def test_no_alloc_leaves_the_device_memory_accounting_unchanged():
    """What the name promises: with the outputs allocated beforehand and the scratch already looked up (first
    call), a call neither takes nor returns device memory. Free memory as the driver reports it, and what the
    framework's allocator has reserved, are the same before and after."""
    x = (torch.randn(2048, 1024, device="cuda") * 2.0).bfloat16()
    qt = torch.empty((1024, 2048), dtype=torch.int8, device="cuda")
    scale = torch.empty((1024, 1), dtype=torch.bfloat16, device="cuda")
    lib, stream = nv.load(), nv.stream_ptr(x.device)

    def call():
        nv.check(lib.qt_quantize_colwise_t_noalloc(x.data_ptr(), nv.QT_BF16, 2048, 1024, 1024, qt.data_ptr(), nv.QT_I8,
                                                   scale.data_ptr(), nv.QT_BF16, 1e-12, 0, 0, 0, stream))

    call()                                   # the first call on a device looks the scratch address up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    want_q, want_s = _two_call_form(x)
    assert torch.equal(qt, want_q) and torch.equal(scale, want_s)
