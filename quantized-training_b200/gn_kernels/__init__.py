"""gn_kernels: the reference's kernel package name, re-hosted on hand-written sm_100a CUDA.

Ops of the hot path keep the reference's names and signatures (kernels/gn_kernels/__init__.py:1-25).
Ops outside it (int4, fp4, conv2d, MX/NVFP4 utilities) raise NotImplementedError.
"""
from .mm import bf16_mm_colscale, bf16_mm_colscale_supported, int8_mm, scaled_mm, scaled_mm_t
from .quantize import (
    col_absmax,
    int8_weight_update_,
    int8_weight_update_supported,
    next_philox_key,
    quantize_colwise,
    quantize_colwise_t,
    quantize_rowwise,
    quantize_rowwise_colabsmax,
    quantize_tile,
)
from ._lib import lib, lib_ops
from . import fused


def _out_of_scope(name: str):
    def fn(*args, **kwargs):
        raise NotImplementedError(
            f"gn_kernels.{name} is outside the INT8/FP8 quantize + scaled GEMM path this build covers"
        )

    fn.__name__ = name
    return fn


int4_mm = _out_of_scope("int4_mm")
scaled_int4_mm = _out_of_scope("scaled_int4_mm")
mxfp4_mm = _out_of_scope("mxfp4_mm")
nvfp4_mm = _out_of_scope("nvfp4_mm")
_triton_conv2d = _out_of_scope("_triton_conv2d")
int8_conv2d = _out_of_scope("int8_conv2d")
scaled_int8_conv2d = _out_of_scope("scaled_int8_conv2d")
quantize_mx = _out_of_scope("quantize_mx")
quantize_nvfp4 = _out_of_scope("quantize_nvfp4")
quantize_nvfp4_triton = _out_of_scope("quantize_nvfp4_triton")
dequantize_mxfp4 = _out_of_scope("dequantize_mxfp4")
pack_block_scales_nv = _out_of_scope("pack_block_scales_nv")
_triton_mm = _out_of_scope("_triton_mm")


def scaled_fp8_mm(A, B, scale_A, scale_B):
    """Row/column-scaled FP8 GEMM (reference: kernels/gn_kernels/cutlass_mm.py scaled_fp8_mm, fp32
    scales, bf16 out). Runs the same tcgen05 kind::f8f6f4 kernel as scaled_mm."""
    import torch

    out = scaled_mm(A, B, scale_A.float().contiguous(), scale_B.float().contiguous())
    return out.to(torch.bfloat16)


def fp8_mm(A, B):
    """Plain FP8 GEMM with bf16 output (reference: cutlass_mm.py fp8_mm): unit scales."""
    import torch

    ones_m = torch.ones((A.shape[0], 1), dtype=torch.bfloat16, device=A.device)
    ones_n = torch.ones((1, 1), dtype=torch.bfloat16, device=A.device)
    return scaled_mm(A, B, ones_m, ones_n)


__all__ = [
    "int4_mm", "scaled_int4_mm", "scaled_fp8_mm", "fp8_mm", "mxfp4_mm", "nvfp4_mm",
    "_triton_conv2d", "int8_conv2d", "scaled_int8_conv2d",
    "_triton_mm", "int8_mm", "scaled_mm",
    "quantize_mx", "quantize_nvfp4", "quantize_nvfp4_triton", "dequantize_mxfp4", "pack_block_scales_nv",
    # quantize kernels (additions; the reference does this step in eager PyTorch)
    "quantize_rowwise", "quantize_rowwise_colabsmax", "col_absmax", "quantize_colwise_t", "quantize_tile",
    "next_philox_key",
]
