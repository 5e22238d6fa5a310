"""Model-level glue with the reference's entry points (train_utils.py:21-75): `quantize_model`
selects a weight subclass by name, `get_optimizer` resolves an optimizer by dotted name,
`get_grad_norm` is the global gradient norm. Only what the INT8 path needs is resolved here; the
reference's bitsandbytes / torchao optimizers are not part of this build."""
from __future__ import annotations

import types
from copy import deepcopy
from functools import partial

import torch
from torch import nn

import other_optim
from subclasses import (
    Int8QTConfig,
    MixedPrecisionConfig,
    convert_bitnet,
    convert_int8_quantized_training,
    convert_mixed_precision,
)


@torch.no_grad()
def get_grad_norm(model: nn.Module) -> float:
    total = sum(p.grad.float().square().sum() for p in model.parameters() if p.grad is not None)
    if hasattr(total, "full_tensor"):
        total = total.full_tensor()
    return float(total) ** 0.5


def get_optimizer(optim: str, model: nn.Module, lr: float, weight_decay: float, **kwargs):
    """`optim` is a dotted expression such as "other_optim.AdamWBF16SR" or "torch.optim.AdamW",
    evaluated against an allow-list (reference: train_utils.py:29-32)."""
    allowed = dict(torch=torch, other_optim=other_optim, partial=partial)
    optim_cls = eval(optim, {"__builtins__": {}}, allowed)
    return optim_cls(model.parameters(), lr=lr, weight_decay=weight_decay, **kwargs)


def _bitnet_rmsnorm_patch(module: nn.Module) -> None:
    """BitNet wants an RMSNorm in front of every quantized Linear (reference: train_utils.py:48-71):
    q/k/v and gate/up inherit the layer's norms, o_proj and down_proj get fresh ones."""
    try:
        from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRMSNorm
    except ImportError:  # no transformers: nothing to patch
        return
    if not isinstance(module, LlamaDecoderLayer):
        return
    attn, mlp = module.self_attn, module.mlp
    for name in ("q_proj", "k_proj", "v_proj"):
        setattr(attn, name, nn.Sequential(deepcopy(module.input_layernorm), getattr(attn, name)))
    for name in ("gate_proj", "up_proj"):
        setattr(mlp, name, nn.Sequential(deepcopy(module.post_attention_layernorm), getattr(mlp, name)))
    ref = module.input_layernorm.weight
    eps = module.input_layernorm.variance_epsilon
    attn.o_proj = nn.Sequential(LlamaRMSNorm(attn.o_proj.in_features, eps).to(device=ref.device, dtype=ref.dtype), attn.o_proj)
    mlp.down_proj = nn.Sequential(LlamaRMSNorm(mlp.down_proj.in_features, eps).to(device=ref.device, dtype=ref.dtype), mlp.down_proj)
    module.input_layernorm = nn.Identity()
    module.post_attention_layernorm = nn.Identity()


def quantize_model(model: nn.Module, quantize: str | None, **kwargs) -> nn.Module:
    """"mixed_precision" | "int8_quantized_training" | "bitnet" | None, with the config fields as
    keyword arguments (reference: train_utils.py:35-75)."""
    if quantize == "mixed_precision":
        convert_mixed_precision(model, config=MixedPrecisionConfig(**kwargs))
    elif quantize == "int8_quantized_training":
        convert_int8_quantized_training(model, config=Int8QTConfig(**kwargs))
    elif quantize == "bitnet":
        model.apply(_bitnet_rmsnorm_patch)
        convert_bitnet(model, **kwargs)
    elif quantize is not None:
        raise ValueError(f"unknown quantization {quantize!r}")
    return model


# ---- element-wise kernels of a Llama-style decoder block -----------------------------------------------


def _is_int8_mixed(linear) -> bool:
    from subclasses.mixed_precision import MixedPrecisionLinearWeight

    w = getattr(linear, "weight", None)
    return isinstance(w, MixedPrecisionLinearWeight) and w.config.dtype == "int8" and w.config.output and not w.config.stochastic_rounding


def fuse_decoder_elementwise(model: nn.Module) -> nn.Module:
    """Replace the element-wise pieces of every Llama-style decoder block under `model` by the single-pass
    kernels of `gn_kernels.fused`: RMSNorm modules, the MLP's silu(gate) * up, and rotary position embedding.
    Call it after `quantize_model`: where the linear layers fed by a norm or by the gated activation are INT8
    mixed precision (round-to-nearest), the producer kernel also emits the quantized activation, so those
    layers skip their own quantize pass (the fusion named at subclasses/int8.py:155-156 of the reference).
    Inputs the kernels do not take (other dtypes, odd shapes) go through the module's original code.
    The reference patches modules in the same manner for BitNet (train_utils.py:48-71)."""
    from gn_kernels import fused

    def norm_forward(self, hidden_states):
        if fused.producer_supported(hidden_states) and self.weight.dtype is torch.bfloat16 and not torch.compiler.is_compiling():
            return fused.rmsnorm(hidden_states, self.weight, self.variance_epsilon, emit_quant=self._qt_emit_quant)
        return self._qt_original_forward(hidden_states)

    def mlp_forward(self, x):
        gate, up = self.gate_proj(x), self.up_proj(x)
        if fused.producer_supported(gate) and up.dtype is torch.bfloat16 and not torch.compiler.is_compiling():
            return self.down_proj(fused.silu_mul(gate, up, emit_quant=self._qt_emit_quant))
        return self.down_proj(self.act_fn(gate) * up)

    def patch_norm(norm: nn.Module, emit_quant: bool):
        if norm is None or not hasattr(norm, "weight") or not hasattr(norm, "variance_epsilon") or hasattr(norm, "_qt_original_forward"):
            return
        norm._qt_original_forward = norm.forward
        norm._qt_emit_quant = emit_quant
        norm.forward = types.MethodType(norm_forward, norm)

    for module in model.modules():
        attn, mlp = getattr(module, "self_attn", None), getattr(module, "mlp", None)
        if attn is not None and mlp is not None and hasattr(module, "input_layernorm"):
            qkv = [getattr(attn, n, None) for n in ("q_proj", "k_proj", "v_proj")]
            patch_norm(module.input_layernorm, all(l is not None and _is_int8_mixed(l) for l in qkv))
            gu = [getattr(mlp, n, None) for n in ("gate_proj", "up_proj")]
            patch_norm(getattr(module, "post_attention_layernorm", None), all(l is not None and _is_int8_mixed(l) for l in gu))
            act = getattr(mlp, "act_fn", None)
            if all(hasattr(mlp, n) for n in ("gate_proj", "up_proj", "down_proj")) and "silu" in type(act).__name__.lower() and not hasattr(mlp, "_qt_emit_quant"):
                mlp._qt_emit_quant = _is_int8_mixed(mlp.down_proj)
                mlp.forward = types.MethodType(mlp_forward, mlp)
    for name in ("norm",):   # the final norm feeds the (unquantized) LM head
        inner = getattr(model, "model", model)
        patch_norm(getattr(inner, name, None), False)

    try:   # rotary embedding: the attention module calls this function by its module-level name
        from transformers.models.llama import modeling_llama
    except ImportError:
        return model
    if not hasattr(modeling_llama, "_qt_original_rope"):
        original = modeling_llama.apply_rotary_pos_emb
        modeling_llama._qt_original_rope = original

        def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
            # q, k arrive as [batch, heads, seq, dim] views of [batch, seq, heads, dim] projections
            if unsqueeze_dim == 1 and q.ndim == 4 and not torch.compiler.is_compiling():
                qt, kt = q.transpose(1, 2), k.transpose(1, 2)
                if fused.rope_supported(qt, cos, sin) and fused.rope_supported(kt, cos, sin):
                    return fused.rope(qt, cos, sin).transpose(1, 2), fused.rope(kt, cos, sin).transpose(1, 2)
            return original(q, k, cos, sin, unsqueeze_dim)

        modeling_llama.apply_rotary_pos_emb = apply_rotary_pos_emb
    return model
