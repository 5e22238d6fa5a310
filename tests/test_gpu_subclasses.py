"""GPU parity of the drop-in tensor subclasses and the optimizer against the reference's recorded
outputs (tests/golden) and the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import reference_math as om
from tests.helpers import bits_of, randn_bf16, values_of

pytestmark = pytest.mark.gpu

import gn_kernels  # noqa: E402
from other_optim import AdamWBF16SR  # noqa: E402
from other_optim.bf16_sr import adamw, adamw_multi  # noqa: E402
from subclasses import (  # noqa: E402
    BitNetTrainingLinearWeight,
    Int8LinearWeight,
    Int8QTConfig,
    MixedPrecisionConfig,
    MixedPrecisionLinearWeight,
    convert_bitnet,
    convert_int8_quantized_training,
    convert_mixed_precision,
)
from subclasses.bitnet import (  # noqa: E402
    BitNetPacked2bitLinearWeight,
    _pack_i2_in_i8,
    _unpack_i2_in_i8,
    get_bitnet_scale,
    quantize_and_pack_bitnet_weight,
    quantize_bitnet_weight,
)
from subclasses.mixed_precision import Int8RowScaledLinearWeight, _dynamic_int8_mm  # noqa: E402


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).cuda()


def test_mixed_precision_linear_matches_reference_recording(golden_dir):
    """forward, grad_input, grad_weight, grad_bias of a converted nn.Linear: bit-exact against what
    the reference's subclass produced on CPU (int8 paths are deterministic)."""
    g = np.load(golden_dir / "mp_linear.npz")
    lin = torch.nn.Linear(192, 160, bias=True).bfloat16().cuda()
    with torch.no_grad():
        lin.weight.copy_(bf16_from_bits(g["w"]))
        lin.bias.copy_(bf16_from_bits(g["b"]))
    convert_mixed_precision(lin, config=MixedPrecisionConfig())
    assert isinstance(lin.weight, MixedPrecisionLinearWeight)
    x = bf16_from_bits(g["x"]).requires_grad_()
    y = lin(x)
    y.backward(bf16_from_bits(g["gy"]))
    np.testing.assert_array_equal(bits_of(y), g["y"])
    np.testing.assert_array_equal(bits_of(x.grad), g["gx"])
    np.testing.assert_array_equal(bits_of(lin.weight.grad), g["gw"])
    np.testing.assert_array_equal(bits_of(lin.bias.grad), g["gb"])
    dyn = _dynamic_int8_mm(x.detach().view(-1, 192), lin.weight._data.T, False)
    np.testing.assert_array_equal(bits_of(dyn), g["dyn"].reshape(dyn.shape))


@pytest.mark.parametrize("cfg", [MixedPrecisionConfig(True, False, False), MixedPrecisionConfig(True, True, False),
                                 MixedPrecisionConfig(False, True, True), MixedPrecisionConfig(True, True, True, "int8", True)])
def test_mixed_precision_config_switches(cfg):
    """Each GEMM can be switched to bf16; results stay within the INT8 quantization error of the
    bf16 linear (1e-2 relative on the norm), and stochastic rounding runs."""
    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 384, bias=False).bfloat16().cuda()
    ref = torch.nn.Linear(256, 384, bias=False).bfloat16().cuda()
    ref.load_state_dict(lin.state_dict())
    convert_mixed_precision(lin, config=cfg)
    x = randn_bf16((4, 64, 256), seed=1)
    x1, x2 = x.clone().requires_grad_(), x.clone().requires_grad_()
    y1, y2 = lin(x1), ref(x2)
    gy = randn_bf16(tuple(y1.shape), seed=2)
    y1.backward(gy)
    y2.backward(gy)
    for a, b in ((y1, y2), (x1.grad, x2.grad), (lin.weight.grad, ref.weight.grad)):
        rel = (a.float() - b.float()).norm() / b.float().norm()
        assert rel < 3e-2, rel


def test_mixed_precision_weight_behaves_like_a_tensor():
    w = randn_bf16((64, 128), seed=3)
    mp = MixedPrecisionLinearWeight(w.clone(), MixedPrecisionConfig())
    assert isinstance(mp.detach(), MixedPrecisionLinearWeight) and isinstance(mp.clone(), MixedPrecisionLinearWeight)
    assert isinstance(mp[:16], MixedPrecisionLinearWeight) and isinstance(mp.view(128, 64), MixedPrecisionLinearWeight)
    assert not isinstance(mp + 1, MixedPrecisionLinearWeight)
    mp.copy_(torch.zeros_like(w))
    assert float(mp._data.abs().sum()) == 0
    names, attrs = mp.__tensor_flatten__()
    again = MixedPrecisionLinearWeight.__tensor_unflatten__({"_data": mp._data}, attrs)
    assert again.config == mp.config and names == ["_data"]
    sd = torch.nn.Linear(128, 64, bias=False).bfloat16().cuda()
    convert_mixed_precision(sd)
    state = sd.state_dict()
    sd.load_state_dict(state)


def test_int8_gathered_weight_forward_backward():
    """The FSDP-gathered form: forward equals the dynamic INT8 matmul of the bf16 weight (row-wise
    quantize commutes with row sharding); backward stays within quantization error."""
    torch.manual_seed(0)
    w = randn_bf16((384, 256), std=0.05, seed=4)
    x = randn_bf16((128, 256), seed=5)
    # quantize two row shards separately, as two FSDP ranks would, and concatenate
    q0, s0 = gn_kernels.quantize_rowwise(w[:192])
    q1, s1 = gn_kernels.quantize_rowwise(w[192:])
    qf, sf = gn_kernels.quantize_rowwise(w)
    assert torch.equal(torch.cat([q0, q1]), qf) and torch.equal(torch.cat([s0, s1]), sf)
    gathered = Int8RowScaledLinearWeight(qf, sf, MixedPrecisionConfig())
    mp = MixedPrecisionLinearWeight(w.clone(), MixedPrecisionConfig())
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya = F.linear(xa, gathered)
    yb = F.linear(xb, mp)
    assert torch.equal(ya, yb)
    gy = randn_bf16(tuple(ya.shape), seed=6)
    # backward with only the forward's (row-wise) quantization at hand: within quantization error
    ya.backward(gy)
    ref_gx = gy.float() @ w.float()
    assert (xa.grad.float() - ref_gx).norm() / ref_gx.norm() < 3e-2
    # the unsharded layer's backward is the reference for the column-wise backward gather
    yb.backward(gy)
    # backward gather: two shards quantized along the output dimension with the agreed column maxima
    colmax = torch.maximum(gn_kernels.col_absmax(w[:192]), gn_kernels.col_absmax(w[192:]))
    assert torch.equal(colmax, gn_kernels.col_absmax(w))
    c0, cs0 = gn_kernels.quantize_colwise(w[:192], colmax)
    c1, cs1 = gn_kernels.quantize_colwise(w[192:], colmax)
    qt_full, cs_full = gn_kernels.quantize_colwise_t(w)
    assert torch.equal(torch.cat([c0, c1]).T.contiguous(), qt_full) and torch.equal(cs0, cs_full) and torch.equal(cs1, cs_full)
    gathered2 = Int8RowScaledLinearWeight(qf.clone(), sf, MixedPrecisionConfig())
    xc = x.clone().requires_grad_()
    yc = F.linear(xc, gathered2)
    assert torch.equal(yc, yb)
    with torch.autograd._unsafe_preserve_version_counter(gathered2.int_data):   # FSDP2 refills the same buffers this way
        gathered2.int_data.copy_(torch.cat([c0, c1]))
    gathered2.mode, gathered2.col_scale = "col", cs0
    yc.backward(gy)
    assert torch.equal(xc.grad, xb.grad)                 # grad_input: bit-identical to the unsharded layer
    # hooks: pre returns int8 rows + scales, post rebuilds the gathered weight
    (wi8, wsc), meta = mp.fsdp_pre_all_gather(None)
    assert wi8.dtype is torch.int8 and torch.equal(wi8, qf) and torch.equal(wsc, sf)
    rebuilt, inner = mp.fsdp_post_all_gather((wi8, wsc), meta, torch.bfloat16)
    assert isinstance(rebuilt, Int8RowScaledLinearWeight) and inner[0] is wi8 and rebuilt.mode == "row"


def test_int8_weight_only_subclass(golden_dir):
    g = np.load(golden_dir / "int8_weight.npz")
    w = bf16_from_bits(g["w"])
    qw = Int8LinearWeight.from_float(w)
    np.testing.assert_array_equal(qw.int_data.cpu().numpy(), g["int_data"])
    np.testing.assert_array_equal(bits_of(qw.scale), g["scale"])
    np.testing.assert_array_equal(bits_of(qw.dequantize()), g["deq"])
    # forward / backward (weight-only): bf16 matmul against the de-quantized weight
    lin = torch.nn.Linear(40, 24, bias=True).bfloat16().cuda()
    with torch.no_grad():
        lin.weight.copy_(w)
    convert_int8_quantized_training(lin)
    x = randn_bf16((8, 40), seed=7).requires_grad_()
    y = lin(x)
    want = (x.detach().float() @ qw.dequantize().float().T) + lin.bias.float()
    assert torch.allclose(y.float(), want, rtol=2e-2, atol=2e-2)
    y.sum().backward()
    assert lin.weight.grad.shape == (24, 40) and x.grad.shape == (8, 40)
    # optimizer path: add_ / addcdiv_ de-quantize, update and re-quantize with stochastic rounding
    p = lin.weight
    before = p.detach().dequantize().float()
    with torch.no_grad():
        p.add_(torch.full((24, 40), 0.25, dtype=torch.bfloat16, device="cuda"))
    after = p.detach().dequantize().float()
    step = (p.detach().scale.float().max()).item()
    assert ((after - before - 0.25).abs() <= 2.5 * step).all()
    assert torch.zeros_like(p).__class__ is torch.Tensor


@pytest.mark.parametrize("act", ["int8", "int8_sr"])
def test_int8_weight_dynamic_activation(act):
    """The call site that is stale in the reference (scale passed as [N,1]) runs here."""
    lin = torch.nn.Linear(256, 128, bias=False).bfloat16().cuda()
    w = lin.weight.detach().clone()
    convert_int8_quantized_training(lin, config=Int8QTConfig(act))
    x = randn_bf16((64, 256), seed=8)
    y = lin(x)
    want = x.float() @ w.float().T
    assert (y.float() - want).norm() / want.norm() < 3e-2


def test_bitnet_helpers_match_reference_recording(golden_dir):
    g = np.load(golden_dir / "bitnet.npz")
    w = bf16_from_bits(g["w"])
    scale = get_bitnet_scale(w)
    assert scale.dtype is torch.float32 and scale.ndim == 0
    assert abs(scale.item() - float(g["scale"])) <= 1e-6 * float(g["scale"])
    ref_scale = torch.tensor(float(g["scale"]), device="cuda")
    wq = quantize_bitnet_weight(w, ref_scale)
    np.testing.assert_array_equal(wq.cpu().numpy(), g["wq"])
    np.testing.assert_array_equal(_pack_i2_in_i8(wq).cpu().numpy(), g["packed"])
    np.testing.assert_array_equal(quantize_and_pack_bitnet_weight(w, ref_scale).cpu().numpy(), g["packed"])
    np.testing.assert_array_equal(_unpack_i2_in_i8(torch.from_numpy(g["packed"]).cuda()).cpu().numpy(), g["unpacked"])
    # every byte value unpacks like the oracle
    allb = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).view(1, -1).cuda()
    np.testing.assert_array_equal(_unpack_i2_in_i8(allb).cpu().numpy(), om.unpack_i2(allb.cpu().numpy()))


def test_bitnet_linear_forward_backward():
    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 192, bias=False).bfloat16().cuda()
    w = lin.weight.detach().clone()
    convert_bitnet(lin)
    assert isinstance(lin.weight, BitNetTrainingLinearWeight)
    x = randn_bf16((96, 256), seed=9).requires_grad_()
    y = lin(x)
    # oracle: int8 activation (eps 1e-5) x ternary weight, row scale x tensor scale
    xq, xs = om.quantize_rowwise(values_of(x), eps=1e-5)
    sc = get_bitnet_scale(w)
    wq = om.bitnet_quantize_weight(values_of(w), np.float32(sc.item()))
    want = om.scaled_mm(xq, wq.T, xs, om.round_to_bf16(np.float32([[sc.item()]])))
    np.testing.assert_array_equal(values_of(y), want)
    y.sum().backward()
    assert x.grad.shape == x.shape and lin.weight.grad.shape == w.shape
    # the packed (gathered) form gives the same forward
    packed = BitNetPacked2bitLinearWeight(quantize_and_pack_bitnet_weight(w, sc), sc.to(torch.bfloat16))
    y2 = F.linear(x.detach(), packed)
    assert torch.equal(y2, y.detach())


@pytest.mark.parametrize("tag", ["sr", "rn"])
def test_adamw_kernel_matches_reference_recording(golden_dir, tag):
    g = np.load(golden_dir / "adamw_bf16_sr.npz")
    step, lr, b1, b2, wd, eps = g["hyper"].tolist()
    p, grad, m, v = (bf16_from_bits(g[f"{tag}_{k}"]) for k in "pgmv")
    if tag == "rn":
        p = p.float()
    # with the reference's random bits unavailable in-kernel, check SR against the oracle's Philox
    key = (1234, 5)
    adamw(p, grad, torch.tensor(step), m, v, torch.tensor(lr), b1, b2, wd, eps, tag == "sr", key=key)
    np.testing.assert_array_equal(bits_of(m), g[f"{tag}_m_out"])
    np.testing.assert_array_equal(bits_of(v), g[f"{tag}_v_out"])
    if tag == "rn":
        np.testing.assert_array_equal(p.cpu().numpy(), g["rn_p_out"])
    else:
        n = p.numel()
        words = om.philox4x32_10(np.arange((n + 3) // 4, dtype=np.uint64), key[1], key[0]).reshape(-1)[:n]
        po, gi, mi, vi = (om.bf16_bits_to_f32(g[f"sr_{k}"]) for k in "pgmv")
        want_p, _, _ = om.adamw_bf16_sr(po, gi, step, mi, vi, lr, b1, b2, wd, eps, words & 0xFFFF)
        np.testing.assert_array_equal(bits_of(p), om.f32_to_bf16_bits(want_p))
        # and the recorded reference result is one of the two bf16 neighbours of the fp32 update
        exact = om.adamw_bf16_sr(po, gi, step, mi, vi, lr, b1, b2, wd, eps, np.zeros(n, np.uint32))[0]
        lo = exact.view(np.uint32) >> 16
        got = bits_of(p).astype(np.uint32)
        assert ((got == lo) | (got == lo + 1)).all()


def test_adamw_stochastic_rounding_is_unbiased():
    n = 1 << 20
    p0 = torch.full((n,), 1.0, dtype=torch.bfloat16, device="cuda")
    g = torch.full((n,), 1e-3, dtype=torch.bfloat16, device="cuda")
    outs = []
    for i in range(4):
        p = p0.clone()
        m = torch.zeros_like(p)
        v = torch.zeros_like(p)
        adamw(p, g, torch.tensor(1.0), m, v, torch.tensor(1e-3), 0.9, 0.999, 0.0, 1e-8, True, key=(9, i))
        outs.append(p.float())
    mean = torch.stack(outs).mean().item()
    # the fp32 update is 1 - 1e-3 (Adam's first step moves by lr); bf16 spacing near 1 is 2^-7 below
    assert abs(mean - (1 - 1e-3)) < 2e-5
    assert len(torch.unique(outs[0])) == 2


@pytest.mark.parametrize("shape", [(3, 8), (257, 264), (1024, 1024), (384, 1536), (96, 5632), (40, 12288), (9, 32768)])
@pytest.mark.parametrize("mode", ["add", "addcdiv"])
def test_fused_int8_weight_update_equals_three_steps(shape, mode):
    """The fused kernel against the reference's own sequence run with eager CUDA ops: de-quantize,
    add_/addcdiv_ on the bf16 tensor, stochastic row-wise re-quantize with the same Philox key."""
    import gn_kernels

    w = randn_bf16(shape, seed=1) * 0.05
    w[0].zero_()                                         # an all-zero row keeps scale 0
    q, scale = gn_kernels.quantize_rowwise(w)
    t1 = randn_bf16(shape, seed=2) * 0.01
    t2 = (randn_bf16(shape, seed=3).abs() * 0.1 + 1e-3).to(torch.bfloat16)
    key = (4321, 17)
    value = -3e-2
    ref = q * scale.view(-1, 1)
    assert ref.dtype is torch.bfloat16
    if mode == "add":
        ref.add_(t1, alpha=value)
    else:
        ref.addcdiv_(t1, t2, value=value)
    want_q, want_s = gn_kernels.quantize_rowwise(ref, torch.int8, True, key=key)
    assert gn_kernels.int8_weight_update_supported(q, scale, t1, t2)
    gn_kernels.int8_weight_update_(q, scale, t1, None if mode == "add" else t2, value, key=key)
    assert torch.equal(scale.view(-1), want_s.view(-1))
    assert torch.equal(q, want_q)


def test_int8_weight_optimizer_step_uses_the_fused_update(monkeypatch):
    import gn_kernels

    calls = []
    real = gn_kernels.int8_weight_update_
    monkeypatch.setattr(gn_kernels, "int8_weight_update_", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    lin = torch.nn.Linear(256, 128, bias=False).bfloat16().cuda()
    convert_int8_quantized_training(lin)
    before = lin.weight.detach().dequantize().float()
    opt = torch.optim.AdamW(lin.parameters(), lr=1e-2, weight_decay=0.0, foreach=False)
    x = randn_bf16((64, 256), seed=5)
    lin(x).float().square().mean().backward()
    opt.step()
    assert calls, "the optimizer's addcdiv_ did not reach the fused kernel"
    after = lin.weight.detach().dequantize().float()
    # Adam's first step moves every weight with a non-zero gradient by about lr
    moved = (after - before).abs()
    assert 0.5e-2 < moved.mean().item() < 2e-2


@pytest.mark.parametrize("p_dtype,g_dtype,sr", [(torch.bfloat16, torch.bfloat16, True), (torch.bfloat16, torch.float32, True),
                                                (torch.float32, torch.bfloat16, False), (torch.float32, torch.float32, False)])
def test_adamw_multi_equals_per_tensor_calls(p_dtype, g_dtype, sr):
    # sizes around the kernel's chunk (8192 elements) and table limit (160 tensors per launch), ragged
    # tails, an empty tensor
    sizes = [1, 3, 4, 7, 0, 8192, 8193, 32768, 65536 + 5, 1000, 4096 * 4096 + 8] + [257 + 4 * i for i in range(180)]
    gen = torch.Generator(device="cuda").manual_seed(3)
    mk = lambda n, dt, scale=1.0: (torch.randn(n, device="cuda", generator=gen) * scale).to(dt)  # noqa: E731
    ps = [mk(n, p_dtype) for n in sizes]
    gs = [mk(n, g_dtype, 0.1) for n in sizes]
    ms = [mk(n, torch.bfloat16, 0.01) for n in sizes]
    vs = [mk(n, torch.bfloat16, 0.01).abs() for n in sizes]
    one = [[t.clone() for t in ts] for ts in (ps, ms, vs)]
    hyper = (torch.tensor(2e-3), 0.9, 0.95, 0.1, 1e-8, sr)
    adamw_multi(ps, gs, 3.0, ms, vs, *hyper, key=(77, 1000))
    for t, (p, g, m, v) in enumerate(zip(one[0], gs, one[1], one[2])):
        if p.numel():
            adamw(p, g, torch.tensor(3.0), m, v, *hyper, key=(77, 1000 + t))
    for got, want in zip(ps + ms + vs, one[0] + one[1] + one[2]):
        assert torch.equal(got, want)
    assert not torch.equal(ps[5], mk(sizes[5], p_dtype))  # the update did something

    # views that start at an odd element (2- or 4-byte aligned only) take the element path: same values
    n = 5000
    base = [mk(n + 1, dt, sc) for dt, sc in ((p_dtype, 1.0), (g_dtype, 0.1), (torch.bfloat16, 0.01), (torch.bfloat16, 0.01))]
    base[3].abs_()
    odd = [t[1:] for t in base]
    even = [t[1:].clone() for t in base]
    adamw_multi([odd[0]], [odd[1]], 3.0, [odd[2]], [odd[3]], *hyper, key=(5, 9))
    adamw(even[0], even[1], torch.tensor(3.0), even[2], even[3], *hyper, key=(5, 9))
    for got, want in zip(odd, even):
        assert torch.equal(got, want)


def test_optimizer_class_trains_a_converted_model():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128, bias=False), torch.nn.ReLU(), torch.nn.Linear(128, 32, bias=False)).bfloat16().cuda()
    convert_mixed_precision(model)
    opt = AdamWBF16SR(model.parameters(), lr=1e-2, weight_decay=0.0)
    x = randn_bf16((256, 64), seed=10)
    target = randn_bf16((256, 32), seed=11)
    losses = []
    for _ in range(30):
        loss = F.mse_loss(model(x).float(), target.float())
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    assert losses[-1] < 0.7 * losses[0]
    st = opt.state[next(iter(model.parameters()))]
    assert st["exp_avg"].dtype is torch.bfloat16 and float(st["step"]) == 30.0
    with pytest.raises(RuntimeError):
        opt.param_groups[0]["lr"] = 1e-3
        loss = F.mse_loss(model(x).float(), target.float())
        loss.backward()
        opt.step()


def test_activation_quantization_cache_is_exact_and_invalidates():
    """A hidden state feeding several projections is quantized once; the cached result must be the
    same bytes, and an in-place update or a new tensor at the same address must miss."""
    from subclasses.int8 import _quant_cache, _rows_quantize

    _quant_cache.clear()
    x = randn_bf16((256, 512), seed=12)
    q1, s1 = _rows_quantize(x, False, 1e-12, cache=True)
    q2, s2 = _rows_quantize(x, False, 1e-12, cache=True)
    assert q2 is q1 and s2 is s1                                  # hit
    x.mul_(2)                                                      # version bump -> miss, fresh values
    q3, s3 = _rows_quantize(x, False, 1e-12, cache=True)
    assert q3 is not q1 and torch.equal(q3, q1) and not torch.equal(s3, s1)
    qt1, _ = _rows_quantize(x.T, False, 1e-12, cache=True)         # transposed view is its own entry
    qt2, _ = _rows_quantize(x.T, False, 1e-12, cache=True)
    assert qt2 is qt1 and qt1.shape == (512, 256)
    qs1, _ = _rows_quantize(x, True, 1e-12, cache=True)            # stochastic rounding is never cached
    qs2, _ = _rows_quantize(x, True, 1e-12, cache=True)
    assert qs1 is not qs2
    # three projections of one input: identical to three independent computations
    lins = [torch.nn.Linear(512, 128, bias=False).bfloat16().cuda() for _ in range(3)]
    for lin in lins:
        convert_mixed_precision(lin)
    _quant_cache.clear()
    with_cache = [lin(x) for lin in lins]
    outs = []
    for lin in lins:
        _quant_cache.clear()
        outs.append(lin(x))
    for a, b in zip(with_cache, outs):
        assert torch.equal(a, b)


def test_real_layer_shape_forward_backward_on_sampled_rows_and_columns():
    """One linear layer of the 1.1B model at the benchmark's token count (32768 x 2048 -> 5632): the oracle is
    evaluated on sampled rows (forward, grad-input: row-wise quantization makes rows independent) and on
    sampled weight entries (grad-weight: columns of the activation and of dY), bit for bit."""
    M, K, N = 32768, 2048, 5632
    x = randn_bf16((M, K), seed=71)
    w = randn_bf16((N, K), std=0.02, seed=72)
    gy = randn_bf16((M, N), std=0.01, seed=73)
    weight = MixedPrecisionLinearWeight(w.clone(), MixedPrecisionConfig()).requires_grad_()
    xr = x.clone().requires_grad_()
    y = F.linear(xr, weight)
    y.backward(gy)
    rows = [0, 1, 4097, 20000, M - 1]
    xs, gs = values_of(x[rows]), values_of(gy[rows])
    wv = values_of(w)
    want_y = om.dynamic_int8_mm(xs, wv.T)
    np.testing.assert_array_equal(values_of(y[rows]), want_y)
    want_gx = om.dynamic_int8_mm(gs, wv)
    np.testing.assert_array_equal(values_of(xr.grad[rows]), want_gx)
    # grad_weight[n, k] = ((x^T dY)^T)[n, k]: needs column k of x and column n of dY over all tokens
    ks, ns = [0, 5, 1023, K - 1], [0, 77, 4000, N - 1]
    xt = values_of(x[:, ks])            # [M, 4]
    gt = values_of(gy[:, ns])           # [M, 4]
    want_gw = om.dynamic_int8_mm(np.ascontiguousarray(xt.T), gt).T      # [4 (n), 4 (k)]
    gw = getattr(weight.grad, "_data", weight.grad)
    assert gw.is_contiguous()                                           # written in the weight's layout, not as a transposed view
    got_gw = values_of(gw)[np.ix_(ns, ks)]
    np.testing.assert_array_equal(got_gw, want_gw)


def test_converted_linear_traces_under_torch_compile_without_freezing_the_noise():
    """The ops carry Meta implementations and the wrappers route through the dispatcher when traced. With the
    `aot_eager` backend (tracing, functionalisation and the autograd split of torch.compile, no code
    generation) a converted Linear gives the eager result bit for bit, forward and backward; with stochastic
    rounding two consecutive calls of the same compiled module differ, i.e. the Philox key is drawn when the op
    runs, not frozen into the graph."""
    torch._dynamo.reset()
    lin = torch.nn.Linear(256, 384, bias=False).bfloat16().cuda()
    convert_mixed_precision(lin, config=MixedPrecisionConfig())
    x = randn_bf16((128, 256), seed=81)
    xe = x.clone().requires_grad_()
    ye = lin(xe)
    ye.float().square().mean().backward()
    ge, gwe = xe.grad.clone(), getattr(lin.weight.grad, "_data", lin.weight.grad).clone()
    lin.weight.grad = None
    compiled = torch.compile(lin, backend="aot_eager", fullgraph=False)
    xc = x.clone().requires_grad_()
    yc = compiled(xc)
    yc.float().square().mean().backward()
    assert torch.equal(yc, ye)
    assert torch.equal(xc.grad, ge)
    assert torch.equal(getattr(lin.weight.grad, "_data", lin.weight.grad), gwe)

    torch._dynamo.reset()
    lin_sr = torch.nn.Linear(256, 384, bias=False).bfloat16().cuda()
    convert_mixed_precision(lin_sr, config=MixedPrecisionConfig(stochastic_rounding=True))
    compiled_sr = torch.compile(lin_sr, backend="aot_eager", fullgraph=False)
    with torch.no_grad():
        a, b = compiled_sr(x), compiled_sr(x)
    assert not torch.equal(a, b)
    assert (a.float() - b.float()).abs().max().item() < 0.1 * a.float().abs().max().item()


def test_converted_model_runs_under_inference_mode_and_the_cache_is_bounded():
    """Tensors made under torch.inference_mode have no version counter: the activation cache must step aside
    (the reference's layer works there). After a backward pass the cache is empty again, and it never holds
    more than its byte cap."""
    from subclasses.int8 import _quant_cache

    lin = torch.nn.Linear(256, 384, bias=False).bfloat16().cuda()
    convert_mixed_precision(lin, config=MixedPrecisionConfig())
    x = randn_bf16((64, 256), seed=91)
    ref = lin(x)
    with torch.inference_mode():
        xi = x.clone()
        out = lin(xi)
    assert torch.equal(out, ref.detach())
    _quant_cache.clear()
    xr = x.clone().requires_grad_()
    y = lin(xr)
    assert len(_quant_cache.entries) >= 1
    y.sum().backward()
    assert len(_quant_cache.entries) == 0
    # the optimizer refuses INT8 weight-only parameters with a clear message
    from other_optim import AdamWBF16SR

    lin8 = torch.nn.Linear(64, 64, bias=False).bfloat16().cuda()
    convert_int8_quantized_training(lin8)
    lin8(randn_bf16((8, 64), seed=3)).sum().backward()
    with pytest.raises(TypeError, match="INT8 weight-only"):
        AdamWBF16SR(lin8.parameters(), lr=1e-3).step()
