"""GPU parity of the absmax quantize kernels: bit-exact int8 / fp8 values and scales against the
CPU oracle and the golden fixtures; stochastic rounding bit-exact against the oracle's Philox
stream and matched in moments against the reference's definition."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import reference_math as om
from tests.helpers import bf16_tensor_from_f32_values, bits_of, randn_bf16, values_of

pytestmark = pytest.mark.gpu

import gn_kernels  # noqa: E402
from gn_kernels import _native as nv  # noqa: E402
from subclasses import quantize_int8  # noqa: E402


def _check_rowwise(x: torch.Tensor, eps=1e-12):
    q, s = gn_kernels.quantize_rowwise(x, eps=eps)
    oq, os_ = om.quantize_rowwise(values_of(x), eps=eps, scale_dtype="bf16" if x.dtype is torch.bfloat16 else "f32")
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    assert s.dtype == x.dtype and s.shape == (x.shape[0], 1)


def test_division_sequence_is_exhaustively_exact():
    """Every (bf16 x, bf16 absmax) pair: the kernels' reciprocal-based division yields the same
    quantized byte as IEEE division (int8 at both eps values the reference uses, and e4m3)."""
    for q_dtype, eps in ((nv.QT_I8, 1e-12), (nv.QT_I8, 1e-5), (nv.QT_E4M3, 1e-12)):
        out = (ctypes.c_ulonglong * 2)(0, 0)
        nv.check(nv.load().qt_selftest_division(q_dtype, eps, out))
        assert out[1] == 0, f"{out[1]} quantized bytes differ (q_dtype={q_dtype}, eps={eps})"


@pytest.mark.parametrize("shape", [(1024, 1024), (333, 777), (64, 4096), (17, 8192), (5, 20000), (3, 40000), (1000, 256),
                                   (129, 2048), (1, 8), (7, 1), (300, 520), (2, 16384), (9, 12288)])
def test_rowwise_matches_oracle(shape):
    _check_rowwise(randn_bf16(shape, seed=shape[0] * 7 + shape[1]))


def test_rowwise_special_rows_and_eps():
    x = randn_bf16((64, 512), seed=3)
    x[0] = 0                      # all-zero row: scale 0, eps clamp
    x[1] = 1e-30                  # below eps * 127
    x[2, 5] = 3.0e38              # near the top of the bf16 range
    x[3] = -x[3].abs()            # all negative
    _check_rowwise(x)
    _check_rowwise(x, eps=1e-5)


def test_rowwise_fp32_input_and_strided_rows():
    g = torch.Generator().manual_seed(5)
    x32 = torch.randn(96, 200, generator=g).cuda()
    _check_rowwise(x32)
    base = randn_bf16((64, 1024), seed=9)
    view = base[:, :512]          # row stride 1024, 512 columns
    q, s = gn_kernels.quantize_rowwise(view)
    oq, os_ = om.quantize_rowwise(values_of(view))
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)


def test_empty_inputs():
    q, s = gn_kernels.quantize_rowwise(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 64) and s.shape == (0, 1)
    q, s = gn_kernels.quantize_rowwise(torch.empty((4, 0), dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (4, 0) and s.shape == (4, 1)


@pytest.mark.parametrize("name", ["bf16_64x96", "bf16_33x257", "bf16_128x1000_small", "bf16_16x2048_eps1e-5", "f32_40x72", "bf16_7x5000"])
def test_quantize_int8_matches_reference_fixtures(golden_dir, name):
    """The drop-in `quantize_int8` against outputs recorded from the reference's function."""
    g = np.load(golden_dir / "quantize.npz")
    for dim in (1, 0):
        xb = g[f"{name}_dim{dim}_x"]
        if xb.dtype == np.uint16:
            x = torch.from_numpy(xb.view(np.int16).copy()).view(torch.bfloat16).cuda()
        else:
            x = torch.from_numpy(xb.copy()).cuda()
        q, s = quantize_int8(x, dim=dim, eps=float(g[f"{name}_dim{dim}_eps"]))
        np.testing.assert_array_equal(q.cpu().numpy(), g[f"{name}_dim{dim}_q"])
        np.testing.assert_array_equal(bits_of(s) if x.dtype is torch.bfloat16 else s.cpu().numpy(), g[f"{name}_dim{dim}_scale"])
        assert q.shape == x.shape and s.shape == g[f"{name}_dim{dim}_scale"].shape


@pytest.mark.parametrize("shape", [(1024, 1024), (333, 777), (4096, 256), (130, 70), (128, 64), (1, 64), (257, 8), (5000, 1024), (2560, 192), (128 * 37, 64)])
def test_colwise_transposed_matches_oracle(shape):
    x = randn_bf16(shape, seed=shape[0] + shape[1])
    qt, s = gn_kernels.quantize_colwise_t(x)
    oq, os_ = om.quantize_colwise_t(values_of(x))
    np.testing.assert_array_equal(qt.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    assert qt.shape == (shape[1], shape[0]) and qt.is_contiguous()
    # the drop-in on a transposed view takes the same route
    q2, s2 = quantize_int8(x.T, dim=1)
    np.testing.assert_array_equal(q2.cpu().numpy(), oq)


def test_fused_rowwise_colabsmax_and_col_absmax():
    for shape in [(512, 1024), (777, 333), (2048, 4096), (100, 8192), (64, 20000)]:
        x = randn_bf16(shape, seed=11 + shape[1])
        q, s, cm = gn_kernels.quantize_rowwise_colabsmax(x)
        oq, os_ = om.quantize_rowwise(values_of(x))
        want_cm = np.abs(values_of(x)).max(axis=0)
        np.testing.assert_array_equal(q.cpu().numpy(), oq)
        np.testing.assert_array_equal(values_of(s), os_)
        np.testing.assert_array_equal(cm.cpu().numpy(), want_cm)
        np.testing.assert_array_equal(gn_kernels.col_absmax(x).cpu().numpy(), want_cm)
        # calling twice reuses nothing stale: the absmax buffer is zeroed per call
        _, _, cm2 = gn_kernels.quantize_rowwise_colabsmax(x * 0.5)
        np.testing.assert_array_equal(cm2.cpu().numpy(), np.abs(values_of(x * 0.5)).max(axis=0))


@pytest.mark.parametrize("shape", [(256, 512), (33, 257), (8, 4096), (64, 20000)])
def test_stochastic_rounding_bit_exact_against_oracle_stream(shape):
    x = randn_bf16(shape, seed=21)
    key = (0x1234_5678_9ABC, 42)
    q, s = gn_kernels.quantize_rowwise(x, stochastic_rounding=True, key=key)
    u = om.philox_uniforms(x.numel(), key[0], key[1]).reshape(shape)
    oq, os_ = om.quantize_rowwise(values_of(x), uniforms=u)
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    # same key, same bytes; another offset, another draw
    q2, _ = gn_kernels.quantize_rowwise(x, stochastic_rounding=True, key=key)
    assert torch.equal(q, q2)
    q3, _ = gn_kernels.quantize_rowwise(x, stochastic_rounding=True, key=(key[0], key[1] + 1))
    assert not torch.equal(q, q3)
    # transposed form draws the uniforms of the transposed element index
    qt, _ = gn_kernels.quantize_colwise_t(x, stochastic_rounding=True, key=key)
    ut = om.philox_uniforms(x.numel(), key[0], key[1]).reshape(shape[1], shape[0])
    oqt, _ = om.quantize_colwise_t(values_of(x), uniforms=ut)
    np.testing.assert_array_equal(qt.cpu().numpy(), oqt)


def test_stochastic_rounding_moments():
    """floor(v + u): unbiased, variance frac * (1 - frac), values in [-128, 127]."""
    x = randn_bf16((2048, 1024), seed=33)
    xv = values_of(x)
    scale = (np.abs(xv).max(axis=1, keepdims=True) / np.float32(127)).astype(np.float32)
    v = (xv / scale).astype(np.float64)
    frac = v - np.floor(v)
    acc = np.zeros_like(v)
    acc2 = np.zeros_like(v)
    n = 16
    for i in range(n):
        q, _ = gn_kernels.quantize_rowwise(x, stochastic_rounding=True, key=(77, i))
        qv = q.cpu().numpy().astype(np.float64)
        assert qv.min() >= -128 and qv.max() <= 127
        err = qv - v
        assert np.abs(err).max() < 1.0 + 1e-4
        acc += err
        acc2 += err * err
    mean_err = acc.sum() / (n * v.size)
    assert abs(mean_err) < 2e-4                                  # ~ 0.29 / sqrt(33M) * 4
    want_var = (frac * (1 - frac)).mean()
    got_var = (acc2 / n).mean()
    assert abs(got_var - want_var) < 2e-3


def test_fp8_rowwise_matches_oracle():
    for shape in [(512, 1024), (33, 257), (16, 8192)]:
        x = randn_bf16(shape, seed=41)
        x[0, :4] = torch.tensor([0.0, -0.0, 1e-20, -1e-20]).bfloat16()
        q, s = gn_kernels.quantize_rowwise(x, out_dtype=torch.float8_e4m3fn)
        oq, os_ = om.quantize_rowwise(values_of(x), out="e4m3")
        np.testing.assert_array_equal(bits_of(q), oq)
        np.testing.assert_array_equal(values_of(s), os_)


def test_tile_quantize_matches_oracle():
    for shape in [(512, 1024), (130, 300), (128, 128), (1000, 2048)]:
        x = randn_bf16(shape, seed=51)
        for tile in ((1, 128), (128, 128)):
            q, s = gn_kernels.quantize_tile(x, tile)
            oq, os_ = om.quantize_tile(values_of(x), tile)
            np.testing.assert_array_equal(q.cpu().numpy(), oq)
            np.testing.assert_array_equal(values_of(s), os_)
        q8, s8 = gn_kernels.quantize_tile(x, (1, 128), out_dtype=torch.float8_e4m3fn)
        oq8, os8 = om.quantize_tile(values_of(x), (1, 128), out="e4m3")
        np.testing.assert_array_equal(bits_of(q8), oq8)


@pytest.mark.parametrize("shape", [(256, 128), (130, 70)])
def test_colwise_saturates_when_the_given_absmax_is_too_small(shape):
    """The column absmax is the caller's: values beyond it saturate at the int8 range (whole-tile and
    ragged shapes take different kernels)."""
    x = randn_bf16(shape, seed=7)
    small = gn_kernels.col_absmax(x) * 0.25
    qt, st = gn_kernels.quantize_colwise_t(x, col_absmax_=small)
    scale = (small.cpu() / 127).view(-1, 1)
    want = torch.clamp(torch.round(x.float().cpu().T / scale.clamp_min(1e-12)), -128, 127).to(torch.int8)
    assert torch.equal(qt.cpu(), want)
    assert (qt == 127).any() and (qt == -128).any()


def test_full_size_properties():
    """Full training sizes (tokens x hidden): size-independent properties instead of an oracle run:
    transposed result == transpose of the column-scaled result, dequantization error bounded by
    half a step, scales == absmax / 127."""
    x = randn_bf16((32768, 2048), seed=61)
    q, s = gn_kernels.quantize_rowwise(x)
    amax = x.float().abs().amax(1, keepdim=True).cpu()
    scale32 = (amax / 127)
    assert torch.equal(s.cpu(), scale32.bfloat16())
    deq_err = (q.float().cpu() * scale32 - x.float().cpu()).abs()
    assert (deq_err <= 0.5 * scale32 * (1 + 1e-3) + 1e-30).all()
    qt, st = gn_kernels.quantize_colwise_t(x)
    cm = gn_kernels.col_absmax(x)
    assert torch.equal(cm.cpu(), x.float().abs().amax(0).cpu())
    assert torch.equal(st.view(-1).cpu(), (cm.cpu() / 127).bfloat16())
    # idempotence on already-quantized values: quantizing q * scale with the same absmax gives q
    deq_err_t = (qt.float().cpu() * (cm.cpu() / 127).view(-1, 1) - x.float().cpu().T).abs()
    assert (deq_err_t <= 0.5 * (cm.cpu() / 127).view(-1, 1) * (1 + 1e-3) + 1e-30).all()


@pytest.mark.parametrize("shape", [(192, 256), (100, 333), (1, 64), (64, 5), (0, 32)])
def test_colwise_without_transpose_matches_oracle(shape):
    """Column-wise scales, rows left in place (the backward weight gather of a row-sharded weight): equal to
    quantize_int8(x, dim=0) of the reference's definition, for bf16 and fp32 input."""
    for dtype in (torch.bfloat16, torch.float32):
        x = randn_bf16(shape, seed=shape[0] + shape[1]).to(dtype)
        colmax = gn_kernels.col_absmax(x)
        q, s = gn_kernels.quantize_colwise(x, colmax)
        assert q.shape == x.shape and s.shape == (shape[1], 1) and s.dtype == dtype
        if shape[0] == 0:
            assert torch.count_nonzero(s) == 0
            continue
        oq, os_ = om.quantize_absmax(values_of(x), axis=0, scale_dtype="bf16" if dtype is torch.bfloat16 else "f32")
        np.testing.assert_array_equal(q.cpu().numpy(), oq)
        np.testing.assert_array_equal(values_of(s).reshape(-1), os_.reshape(-1))


@pytest.mark.parametrize("shape", [(256, 512), (100, 333), (64, 4096)])
def test_rowwise_e5m2_matches_oracle(shape):
    x = randn_bf16(shape, seed=shape[1] + 1)
    q, s = gn_kernels.quantize_rowwise(x, torch.float8_e5m2)
    oq, os_ = om.quantize_rowwise(values_of(x), out="e5m2")
    np.testing.assert_array_equal(bits_of(q), oq)
    np.testing.assert_array_equal(values_of(s), os_)


@pytest.mark.parametrize("shape", [(256, 256), (384, 1024), (130, 200)])
@pytest.mark.parametrize("out", ["e4m3", "e5m2"])
def test_tile_128x128_fp8_matches_oracle(shape, out):
    x = randn_bf16(shape, seed=shape[0] + 3)
    dt = torch.float8_e4m3fn if out == "e4m3" else torch.float8_e5m2
    q, s = gn_kernels.quantize_tile(x, (128, 128), dt)
    oq, os_ = om.quantize_tile(values_of(x), (128, 128), out=out)
    np.testing.assert_array_equal(bits_of(q), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    q1, s1 = gn_kernels.quantize_tile(x, (1, 128), dt)
    oq1, os1 = om.quantize_tile(values_of(x), (1, 128), out=out)
    np.testing.assert_array_equal(bits_of(q1), oq1)
    np.testing.assert_array_equal(values_of(s1), os1)


def test_quantize_kernels_give_the_same_bits_twice():
    x = randn_bf16((4096, 2048), seed=12)
    a = gn_kernels.quantize_rowwise_colabsmax(x)
    b = gn_kernels.quantize_rowwise_colabsmax(x)
    assert all(torch.equal(u, v) for u, v in zip(a, b))
    k = (2024, 5)
    a = gn_kernels.quantize_rowwise(x, torch.int8, True, key=k)
    b = gn_kernels.quantize_rowwise(x, torch.int8, True, key=k)
    assert torch.equal(a[0], b[0])
    c = gn_kernels.quantize_rowwise(x, torch.int8, True, key=(2024, 6))
    assert not torch.equal(a[0], c[0])
