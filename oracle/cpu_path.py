"""The reference's CPU-runnable form of the hot path, restated with torch CPU ops.  TEST / CPU-BASELINE
INFRASTRUCTURE ONLY: imported by the test-suite and by the benchmark's CPU-baseline and
`--impl reference` legs, never by the product packages.

The reference's kernels are CUDA-only; what it can run on a host is its eager `quantize_int8`
(subclasses/int8.py:12-26) followed by `torch._int_mm` and the scale multiply -- the combination
its benchmark uses as the inductor comparator (benchmark_mm.py:37-43) and the path named as the CPU
baseline for this build. This file restates exactly that, op for op, so it can be timed on a box
where the reference checkout is absent. Pinned against the reference by
tests/test_oracle_golden.py::test_cpu_path_matches_reference_fixtures.
"""
from __future__ import annotations

import torch
from torch import Tensor


@torch.no_grad()
def quantize_rows_int8(x: Tensor, eps: float = 1e-12):
    """quantize_int8(x, dim=1), round-to-nearest (subclasses/int8.py:12-26)."""
    xf = x.float()
    scale = xf.abs().amax(1, keepdim=True) / 127
    q = (xf / scale.clip(eps)).round().clip(-128, 127).to(torch.int8)
    return q, scale.to(x.dtype)


@torch.no_grad()
def dynamic_int8_linear(A: Tensor, B: Tensor) -> Tensor:
    """bf16 A [M,K], B [N,K] -> bf16 A @ B.T through row-wise INT8 (the 1024^2, seed-2024 configuration):
    quantize both along K, int32 accumulate with torch._int_mm, de-scale as the Triton epilogue
    does (kernels/gn_kernels/triton_mm.py:210-216)."""
    qa, sa = quantize_rows_int8(A)
    qb, sb = quantize_rows_int8(B)
    acc = torch._int_mm(qa, qb.T)
    return (acc.float() * sa.float() * sb.float().T).to(sa.dtype)
