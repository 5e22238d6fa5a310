"""GPU parity of the producer-fused kernels (RMSNorm + quantize, silu * up + quantize), their backward
passes and rotary position embedding.

The bf16 results are compared with the eager formulas of the model code the reference trains
(transformers' Llama: RMSNorm, act_fn(gate) * up, apply_rotary_pos_emb) evaluated by PyTorch: nearly all
elements identical, the rest one bf16 step apart (fast exponential / different summation order before a
bf16 rounding). The quantized outputs are compared bit for bit with the CPU oracle's quantize_int8 of the
kernel's own bf16 result, which is what the following linear layer would have computed by itself
(reference: subclasses/int8.py:12-26 called at subclasses/mixed_precision.py:100-108)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import reference_math as om
from tests.helpers import randn_bf16, values_of

pytestmark = pytest.mark.gpu

import gn_kernels  # noqa: E402
from gn_kernels import _native as nv  # noqa: E402
from gn_kernels import fused  # noqa: E402

# A bf16 step is at most 2^-7 relative. The few elements that differ (see _mostly_equal) may be two steps
# apart: a one-step difference in the normalised value, multiplied by the weight and rounded again.
ONE_STEP = dict(rtol=2.0 ** -6, atol=1e-30)


def _mostly_equal(a: torch.Tensor, b: torch.Tensor, frac: float = 0.999):
    same = (a == b).float().mean().item()
    assert same >= frac, f"only {same:.5f} of the elements are identical"
    torch.testing.assert_close(a.float(), b.float(), **ONE_STEP)


def _rmsnorm_eager(x, w, eps):
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return w * h.to(x.dtype)


def _call_rmsnorm(x, w, eps, quant=True):
    rows, cols = x.shape
    dev = x.device
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    q = torch.empty(rows, cols, dtype=torch.int8, device=dev)
    s = torch.empty(rows, 1, dtype=torch.bfloat16, device=dev)
    cm = torch.empty(cols, dtype=torch.float32, device=dev)
    nv.check(nv.load().qt_rmsnorm_quantize(x.data_ptr(), rows, cols, x.stride(0), w.data_ptr(), eps, y.data_ptr(), rstd.data_ptr(),
                                           q.data_ptr() if quant else None, nv.QT_I8, s.data_ptr() if quant else None, nv.QT_BF16,
                                           cm.data_ptr() if quant else None, 1e-12, nv.stream_ptr(dev)))
    return y, rstd, q, s, cm


@pytest.mark.parametrize("shape", [(64, 256), (128, 2048), (32, 5632), (8, 16384), (4096, 2048), (16, 1000), (8, 8)])
def test_rmsnorm_quantize_forward(shape):
    x = randn_bf16(shape, seed=shape[1])
    w = (1.0 + 0.1 * torch.randn(shape[1])).bfloat16().cuda()
    y, rstd, q, s, cm = _call_rmsnorm(x, w, 1e-6)
    _mostly_equal(y, _rmsnorm_eager(x, w, 1e-6))
    ref_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    torch.testing.assert_close(rstd, ref_rstd, rtol=1e-5, atol=0)
    # the quantized copy is exactly quantize_int8 of the bf16 result
    oq, os_ = om.quantize_rowwise(values_of(y))
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    np.testing.assert_array_equal(cm.cpu().numpy(), np.abs(values_of(y)).max(axis=0))
    # without the quantized outputs the bf16 result is the same
    y2, *_ = _call_rmsnorm(x, w, 1e-6, quant=False)
    assert torch.equal(y, y2)


def test_rmsnorm_quantize_strided_rows_and_unsupported_shapes():
    base = randn_bf16((64, 1024), seed=4)
    x = base[:, :512]
    w = torch.ones(512, dtype=torch.bfloat16, device="cuda")
    y, _, q, s, _ = _call_rmsnorm(x, w, 1e-5)
    _mostly_equal(y, _rmsnorm_eager(x, w, 1e-5))
    oq, os_ = om.quantize_rowwise(values_of(y))
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    # a row count the row grouping does not divide is refused (the Python layer then runs norm and quantize apart)
    x7 = randn_bf16((7, 512), seed=5)
    with pytest.raises(RuntimeError, match="multiple"):
        _call_rmsnorm(x7, w, 1e-5)
    assert not fused.producer_supported(x7)
    assert fused.producer_supported(x)


@pytest.mark.parametrize("shape", [(64, 256), (256, 2048), (30, 1000), (16, 5632), (4, 16384)])
def test_rmsnorm_backward_matches_autograd(shape):
    x = randn_bf16(shape, seed=11).requires_grad_(True)
    w = (1.0 + 0.1 * torch.randn(shape[1])).bfloat16().cuda().requires_grad_(True)
    dy = randn_bf16(shape, seed=12)
    # fp32 reference of the same function
    x32, w32 = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    n = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-6)
    (w32 * n).backward(dy.float())
    rows = shape[0]
    if fused.producer_supported(x):
        y = fused.rmsnorm(x, w, 1e-6)
        y.backward(dy)
        dx, dw = x.grad, w.grad
    else:   # the backward kernel takes any row count: call it directly
        rstd = torch.rsqrt(x.detach().float().pow(2).mean(-1) + 1e-6)
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        n_partial = nv.load().qt_rmsnorm_backward_partial_rows(rows, shape[1])
        partial = torch.empty(n_partial, shape[1], dtype=torch.float32, device="cuda")
        nv.check(nv.load().qt_rmsnorm_backward(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), rstd.data_ptr(),
                                               rows, shape[1], dx.data_ptr(), partial.data_ptr(), n_partial, dw.data_ptr(), nv.QT_BF16,
                                               nv.stream_ptr(x.device)))
    # north-star tolerance for bf16 results: 1e-2 relative (plus the bf16 rounding floor near zero)
    torch.testing.assert_close(dx.float(), x32.grad, rtol=1e-2, atol=1e-2 * x32.grad.abs().max().item())
    torch.testing.assert_close(dw.float(), w32.grad, rtol=1e-2, atol=1e-2 * w32.grad.abs().max().item())


def test_rmsnorm_backward_is_deterministic():
    x = randn_bf16((2048, 2048), seed=21)
    w = torch.ones(2048, dtype=torch.bfloat16, device="cuda")
    dy = randn_bf16((2048, 2048), seed=22)
    outs = []
    for _ in range(2):
        xx, ww = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        fused.rmsnorm(xx, ww, 1e-6).backward(dy)
        outs.append((xx.grad.clone(), ww.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("shape", [(64, 256), (128, 5632), (32, 2816), (8, 16384), (2048, 1024)])
def test_silu_mul_quantize_forward(shape):
    g, u = randn_bf16(shape, seed=31, std=2.0), randn_bf16(shape, seed=32)
    rows, cols = shape
    y = torch.empty_like(g)
    q = torch.empty(rows, cols, dtype=torch.int8, device="cuda")
    s = torch.empty(rows, 1, dtype=torch.bfloat16, device="cuda")
    cm = torch.empty(cols, dtype=torch.float32, device="cuda")
    nv.check(nv.load().qt_silu_mul_quantize(g.data_ptr(), u.data_ptr(), rows, cols, cols, cols, y.data_ptr(), q.data_ptr(), nv.QT_I8,
                                            s.data_ptr(), nv.QT_BF16, cm.data_ptr(), 1e-12, nv.stream_ptr(g.device)))
    _mostly_equal(y, F.silu(g) * u, frac=0.995)
    oq, os_ = om.quantize_rowwise(values_of(y))
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    np.testing.assert_array_equal(values_of(s), os_)
    np.testing.assert_array_equal(cm.cpu().numpy(), np.abs(values_of(y)).max(axis=0))


def test_silu_mul_extreme_inputs():
    g = torch.tensor([[-200.0, -30.0, -1e-3, 0.0, 1e-3, 30.0, 200.0, 3e4]] * 8, dtype=torch.bfloat16, device="cuda")
    u = torch.full_like(g, 1.5)
    y = fused.silu_mul(g, u)
    ref = F.silu(g) * u
    assert torch.isfinite(y).all()
    torch.testing.assert_close(y.float(), ref.float(), **ONE_STEP)


@pytest.mark.parametrize("shape", [(64, 256), (128, 5632), (33, 1000)])
def test_silu_mul_backward_matches_autograd(shape):
    g, u, dh = randn_bf16(shape, seed=41, std=2.0), randn_bf16(shape, seed=42), randn_bf16(shape, seed=43)
    g32, u32 = g.float().requires_grad_(True), u.float().requires_grad_(True)
    (F.silu(g32) * u32).backward(dh.float())
    dg = torch.empty_like(g)
    du = torch.empty_like(g)
    rows, cols = shape
    nv.check(nv.load().qt_silu_mul_backward(dh.data_ptr(), cols, g.data_ptr(), cols, u.data_ptr(), cols, rows, cols, dg.data_ptr(),
                                            du.data_ptr(), nv.stream_ptr(g.device)))
    torch.testing.assert_close(dg.float(), g32.grad, rtol=1e-2, atol=1e-2 * g32.grad.abs().max().item())
    torch.testing.assert_close(du.float(), u32.grad, rtol=1e-2, atol=1e-2 * u32.grad.abs().max().item())


def _rope_eager(x, cos, sin):
    # x [b, s, h, d]; cos / sin [b or 1, s, d]
    c, s_ = cos.unsqueeze(2), sin.unsqueeze(2)
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return x * c + torch.cat((-x2, x1), dim=-1) * s_


@pytest.mark.parametrize("b,s,h,d,tb", [(2, 64, 4, 64, 1), (3, 128, 32, 64, 3), (1, 256, 2, 128, 1), (2, 16, 5, 32, 2)])
def test_rope_forward_and_backward(b, s, h, d, tb):
    x = randn_bf16((b, s, h, d), seed=51)
    ang = torch.randn(tb, s, d // 2)
    ang = torch.cat((ang, ang), dim=-1)
    cos, sin = ang.cos().bfloat16().cuda(), ang.sin().bfloat16().cuda()
    assert fused.rope_supported(x, cos, sin)
    xr = x.clone().requires_grad_(True)
    y = fused.rope(xr, cos, sin)
    x32 = x.float().requires_grad_(True)
    ref = _rope_eager(x32, cos.float(), sin.float())
    # the eager bf16 form rounds three times, the kernel once: compare with the fp32 evaluation
    torch.testing.assert_close(y.float(), ref, rtol=2.0 ** -8, atol=2.0 ** -8)
    dy = randn_bf16((b, s, h, d), seed=52)
    y.backward(dy)
    ref.backward(dy.float())
    torch.testing.assert_close(xr.grad.float(), x32.grad, rtol=2.0 ** -8, atol=2.0 ** -8 * 4)


def _tiny_llama(seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(seed)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64, attn_implementation="sdpa", tie_word_embeddings=False)
    with torch.device("cuda"):
        return LlamaForCausalLM(cfg).bfloat16()


def test_fused_decoder_block_matches_the_unfused_model_and_feeds_the_linears():
    """A converted tiny Llama with the element-wise kernels swapped in: (1) with and without the parked
    quantized activations the logits are bit-identical (what the producer emits is exactly what the linear
    layers would have computed); (2) loss and gradients agree with the unfused model within the bf16
    tolerance; (3) the linear layers really did skip their quantize (the cache is hit)."""
    import copy

    from subclasses.int8 import _quant_cache
    from train_utils import fuse_decoder_elementwise, quantize_model

    base = _tiny_llama()
    quantize_model(base.model, "mixed_precision")
    tokens = torch.randint(0, 512, (8, 65), device="cuda")

    def run(model):
        model.zero_grad(set_to_none=True)
        logits = model(input_ids=tokens[:, :-1]).logits.float()
        loss = F.cross_entropy(logits.view(-1, 512), tokens[:, 1:].reshape(-1))
        loss.backward()
        grads = {n: p.grad.float().clone() for n, p in model.named_parameters()}
        return logits.detach(), loss.detach(), grads

    ref_logits, ref_loss, ref_grads = run(base)

    fused_model = fuse_decoder_elementwise(copy.deepcopy(base))
    hits = {"n": 0}
    orig_get = _quant_cache.get

    def counting_get(t, eps):
        out = orig_get(t, eps)
        hits["n"] += out is not None
        return out

    _quant_cache.get = counting_get
    try:
        logits, loss, grads = run(fused_model)
    finally:
        _quant_cache.get = orig_get
    # q, k, v + gate, up + down per layer find the producer's quantization (forward) -> at least 6 per layer
    assert hits["n"] >= 12, hits

    plain = fuse_decoder_elementwise(copy.deepcopy(base))
    for m in plain.modules():
        if hasattr(m, "_qt_emit_quant"):
            m._qt_emit_quant = False
    logits2, loss2, grads2 = run(plain)
    assert torch.equal(logits, logits2)
    for n in grads:
        assert torch.equal(grads[n], grads2[n]), n

    torch.testing.assert_close(loss, ref_loss, rtol=1e-2, atol=1e-2)
    for n in ref_grads:
        scale = ref_grads[n].abs().max().item() + 1e-12
        err = (grads[n] - ref_grads[n]).abs().max().item() / scale
        assert err < 0.1, (n, err)
