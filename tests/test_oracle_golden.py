"""Pins the numpy oracle to outputs of the reference project's own functions (the fixtures under
tests/golden, written by tests/golden/make_golden.py). CPU only."""
import hashlib
import json

import numpy as np
import pytest

from oracle import reference_math as om


def _val(a):
    """Fixture arrays hold bf16 as uint16 bit patterns and fp32 as float32."""
    return om.bf16_bits_to_f32(a) if a.dtype == np.uint16 else a.astype(np.float32)


def _bits(values_f32, like):
    return om.f32_to_bf16_bits(values_f32) if like.dtype == np.uint16 else np.asarray(values_f32, dtype=np.float32)


QUANT_CASES = ["bf16_64x96", "bf16_33x257", "bf16_128x1000_small", "bf16_16x2048_eps1e-5", "f32_40x72", "bf16_7x5000"]


@pytest.mark.parametrize("name", QUANT_CASES)
@pytest.mark.parametrize("dim", [1, 0])
def test_quantize_rtne_matches_reference(golden_dir, name, dim):
    g = np.load(golden_dir / "quantize.npz")
    xb = g[f"{name}_dim{dim}_x"]
    x = _val(xb)
    sdt = "bf16" if xb.dtype == np.uint16 else "f32"
    eps = float(g[f"{name}_dim{dim}_eps"])
    q, s = om.quantize_absmax(x, axis=dim, eps=eps, scale_dtype=sdt)
    np.testing.assert_array_equal(q, g[f"{name}_dim{dim}_q"])
    np.testing.assert_array_equal(_bits(s, g[f"{name}_dim{dim}_scale"]), g[f"{name}_dim{dim}_scale"])
    if dim == 0:  # the transposing form used by the kernels
        qt, st = om.quantize_colwise_t(x, eps=eps, scale_dtype=sdt)
        np.testing.assert_array_equal(qt, g[f"{name}_dim0_q"].T)
        np.testing.assert_array_equal(st.reshape(-1), s.reshape(-1))


@pytest.mark.parametrize("name", QUANT_CASES)
def test_quantize_stochastic_matches_reference_given_its_uniforms(golden_dir, name):
    g = np.load(golden_dir / "quantize.npz")
    x = _val(g[f"{name}_dim1_x"])
    eps = float(g[f"{name}_dim1_eps"])
    q, _ = om.quantize_absmax(x, axis=1, eps=eps, uniforms=g[f"{name}_sr_u"])
    np.testing.assert_array_equal(q, g[f"{name}_sr_q"])
    assert q.min() >= -128 and q.max() <= 127


def test_int8_mm_and_scaled_mm_against_reference_functions(golden_dir):
    g = np.load(golden_dir / "scaled_mm_ref.npz")
    A, B = g["A"], g["B"]
    np.testing.assert_array_equal(om.int8_mm(A, B), g["int_mm"])  # benchmark_mm.py:112 demands equality
    sA, sB = _val(g["sA"]), _val(g["sB"])
    out = om.scaled_mm(A, B, sA, sB)
    # tolerances of benchmark_mm.py:116-118
    np.testing.assert_allclose(out, _val(g["rowcol"]), atol=4e-4, rtol=1e-2)
    tile = om.tile_scaled_mm(A, B, _val(g["tsA"]), _val(g["tsB"]))
    # benchmark_mm.py:119-121
    np.testing.assert_allclose(tile, _val(g["tile"]), atol=1e-4, rtol=1e-2)


def test_fp8_paths_against_reference_functions(golden_dir):
    g = np.load(golden_dir / "scaled_mm_ref.npz")
    A8, B8 = g["A8"], g["B8"]
    sA, sB = _val(g["sA"]), _val(g["sB"])
    ones_m, ones_n = np.ones((A8.shape[0], 1), np.float32), np.ones((1, B8.shape[1]), np.float32)
    # default bf16 assert_close tolerances (benchmark_mm.py:129,142-145): rtol 1.6e-2, atol 1e-5
    np.testing.assert_allclose(om.scaled_mm(A8, B8, ones_m, ones_n, kind="e4m3"), _val(g["f8_plain"]), rtol=1.6e-2, atol=1e-5)
    np.testing.assert_allclose(om.scaled_mm(A8, B8, sA, sB, kind="e4m3"), _val(g["f8_rowcol"]), rtol=1.6e-2, atol=1e-5)
    np.testing.assert_allclose(om.tile_scaled_mm(A8, B8, _val(g["tsA"]), _val(g["tsB"]), kind="e4m3"), _val(g["f8_tile"]),
                               rtol=1.6e-2, atol=2e-5)


def test_e4m3_codec_roundtrip_and_rounding():
    codes = np.arange(256, dtype=np.uint8)
    vals = om.e4m3_bits_to_f32(codes)
    finite = ~np.isnan(vals)
    np.testing.assert_array_equal(om.f32_to_e4m3_bits(vals[finite]), codes[finite])
    # ties go to the even code; overflow saturates
    assert om.f32_to_e4m3_bits(np.float32([0.0, 1e9, -1e9, 17.0, 19.0])).tolist() == [0, 0x7E, 0xFE, 0x58, 0x5A]


def test_mixed_precision_linear_forward_backward(golden_dir):
    g = np.load(golden_dir / "mp_linear.npz")
    x = _val(g["x"]).reshape(-1, 192)
    w, b, gy = _val(g["w"]), _val(g["b"]), _val(g["gy"]).reshape(-1, 160)
    dyn = om.mixed_precision_linear_forward(x, w)
    np.testing.assert_array_equal(om.f32_to_bf16_bits(dyn).reshape(-1), g["dyn"].reshape(-1))
    y = om.round_to_bf16(dyn + b[None, :])
    np.testing.assert_array_equal(om.f32_to_bf16_bits(y).reshape(-1), g["y"].reshape(-1))
    gx, gw = om.mixed_precision_linear_backward(x, w, gy)
    np.testing.assert_array_equal(om.f32_to_bf16_bits(gx).reshape(-1), g["gx"].reshape(-1))
    np.testing.assert_array_equal(om.f32_to_bf16_bits(np.ascontiguousarray(gw)).reshape(-1), g["gw"].reshape(-1))


@pytest.mark.parametrize("tag", ["sr", "rn"])
def test_adamw_bf16_sr(golden_dir, tag):
    g = np.load(golden_dir / "adamw_bf16_sr.npz")
    step, lr, b1, b2, wd, eps = g["hyper"].tolist()
    p, grad, m, v = (_val(g[f"{tag}_{k}"]) for k in "pgmv")
    rand = g[f"{tag}_rand"] if tag == "sr" else None
    new_p, new_m, new_v = om.adamw_bf16_sr(p, grad, step, m, v, lr, b1, b2, wd, eps, rand)
    np.testing.assert_array_equal(om.f32_to_bf16_bits(new_m), g[f"{tag}_m_out"])
    np.testing.assert_array_equal(om.f32_to_bf16_bits(new_v), g[f"{tag}_v_out"])
    if tag == "sr":
        np.testing.assert_array_equal(om.f32_to_bf16_bits(new_p), g["sr_p_out"])
    else:
        # fp32 parameter: the reference writes the unrounded fp32 update back
        ref = g["rn_p_out"]
        raw = om.adamw_bf16_sr(p, grad, step, m, v, lr, b1, b2, wd, eps, None)[0]
        np.testing.assert_array_equal(raw, om.round_to_bf16(ref))


def test_bitnet_helpers(golden_dir):
    g = np.load(golden_dir / "bitnet.npz")
    w = _val(g["w"])
    assert abs(float(om.bitnet_scale(w)) - float(g["scale"])) <= 1e-6 * float(g["scale"])
    wq = om.bitnet_quantize_weight(w, g["scale"])
    np.testing.assert_array_equal(wq, g["wq"])
    np.testing.assert_array_equal(om.pack_i2(wq), g["packed"])
    np.testing.assert_array_equal(om.unpack_i2(g["packed"]), g["unpacked"])
    np.testing.assert_array_equal(om.unpack_i2(om.pack_i2(wq)), wq)


def test_int8_weight_fixture(golden_dir):
    g = np.load(golden_dir / "int8_weight.npz")
    q, s = om.quantize_rowwise(_val(g["w"]))
    np.testing.assert_array_equal(q, g["int_data"])
    np.testing.assert_array_equal(om.f32_to_bf16_bits(s), g["scale"])
    deq = om.round_to_bf16(q.astype(np.float32) * s)  # Int8LinearWeight.dequantize, int8.py:60-61
    np.testing.assert_array_equal(om.f32_to_bf16_bits(deq), g["deq"])


def test_config1_digests(golden_dir):
    """The 1024^2, seed-2024 configuration: regenerate the inputs from the seed and compare
    SHA-256 digests of every intermediate with those the reference produced."""
    torch = pytest.importorskip("torch")
    ref = json.loads((golden_dir / "config1_digest.json").read_text())
    torch.manual_seed(2024)
    A = torch.randn(1024, 1024).bfloat16()
    B = (torch.randn(1024, 1024) * 0.02).bfloat16()
    Ab = A.view(torch.int16).numpy().view(np.uint16)
    Bb = B.view(torch.int16).numpy().view(np.uint16)

    def dig(a):
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()

    if dig(Ab) != ref["A"] or dig(Bb) != ref["B"]:
        pytest.skip("this torch build draws different randn values than the one that wrote the fixture")
    qa, sa = om.quantize_rowwise(om.bf16_bits_to_f32(Ab))
    qb, sb = om.quantize_rowwise(om.bf16_bits_to_f32(Bb))
    acc = om.int8_mm(qa, qb.T)
    out = om.scaled_mm(qa, qb.T, sa, sb.T)
    assert dig(qa) == ref["qa"] and dig(qb) == ref["qb"]
    assert dig(om.f32_to_bf16_bits(sa)) == ref["sa"] and dig(om.f32_to_bf16_bits(sb)) == ref["sb"]
    assert dig(acc) == ref["acc"]
    assert dig(om.f32_to_bf16_bits(out)) == ref["out"]
    assert [int(qa.min()), int(qa.max())] == ref["qa_range"]


def test_cpu_path_matches_reference_fixtures(golden_dir):
    """The torch-CPU restatement used as the timed CPU baseline reproduces the reference's digests
    on the 1024^2, seed-2024 configuration and agrees bit-for-bit with the numpy oracle."""
    torch = pytest.importorskip("torch")
    from oracle import cpu_path

    ref = json.loads((golden_dir / "config1_digest.json").read_text())
    torch.manual_seed(2024)
    A = torch.randn(1024, 1024).bfloat16()
    B = (torch.randn(1024, 1024) * 0.02).bfloat16()

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    def dig(a):
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()

    out = cpu_path.dynamic_int8_linear(A, B)
    qa, sa = cpu_path.quantize_rows_int8(A)
    oqa, osa = om.quantize_rowwise(A.float().numpy())
    np.testing.assert_array_equal(qa.numpy(), oqa)
    np.testing.assert_array_equal(sa.float().numpy(), osa)
    oqb, osb = om.quantize_rowwise(B.float().numpy())
    np.testing.assert_array_equal(out.float().numpy(), om.scaled_mm(oqa, oqb.T, osa, osb.T))
    if dig(bits(A)) == ref["A"] and dig(bits(B)) == ref["B"]:
        assert dig(bits(out)) == ref["out"] and dig(qa.numpy()) == ref["qa"]


def test_e5m2_codec_roundtrip_and_rounding():
    """The second FP8 format: decode table, round-to-nearest-even with saturation at 57344, pinned against
    the casts of the framework the reference runs on (torch.float8_e5m2 on CPU)."""
    import torch

    codes = np.arange(256, dtype=np.uint8)
    vals = om.e5m2_bits_to_f32(codes)
    finite = np.isfinite(vals)
    np.testing.assert_array_equal(om.f32_to_e5m2_bits(vals[finite]), codes[finite])
    assert om.f32_to_e5m2_bits(np.float32([0.0, 1e9, -1e9, 57344.0, 1.25, 1.125, 1.375])).tolist() == [0, 0x7B, 0xFB, 0x7B, 0x3D, 0x3C, 0x3E]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(100000, generator=g) * torch.logspace(-7, 4.5, 100000)
    ref = x.clamp(-57344, 57344).to(torch.float8_e5m2).view(torch.uint8).numpy()
    np.testing.assert_array_equal(om.f32_to_e5m2_bits(x.numpy()), ref)
    np.testing.assert_array_equal(np.nan_to_num(vals, nan=7.0), np.nan_to_num(torch.from_numpy(codes).view(torch.float8_e5m2).float().numpy(), nan=7.0))
