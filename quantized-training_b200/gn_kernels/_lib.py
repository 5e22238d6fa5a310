"""The `gn_kernels` operator namespace (same name and schemas as the reference's registry,
kernels/gn_kernels/_lib.py:3-4), backed by libqt_b200.so instead of Triton / CUTLASS."""
import torch

lib = torch.library.Library("gn_kernels", "DEF")
lib_ops = torch.ops.gn_kernels
