"""Model-level glue with the reference's entry points (train_utils.py:21-75): `quantize_model`
selects a weight subclass by name, `get_optimizer` resolves an optimizer by dotted name,
`get_grad_norm` is the global gradient norm. Only what the INT8 path needs is resolved here; the
reference's bitsandbytes / torchao optimizers are not part of this build."""
from __future__ import annotations

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
