"""Shared helpers of the GPU parity tests: torch <-> numpy bridges for bf16 / fp8 bit patterns."""
import numpy as np
import torch

from oracle import reference_math as om


def bf16_tensor_from_f32_values(values: np.ndarray, device="cuda") -> torch.Tensor:
    bits = om.f32_to_bf16_bits(values).view(np.int16)
    return torch.from_numpy(bits.copy()).view(torch.bfloat16).reshape(values.shape).to(device)


def bits_of(t: torch.Tensor) -> np.ndarray:
    """Raw bit patterns of a bf16 / fp8 / int tensor as a numpy array."""
    t = t.detach().contiguous().cpu()
    if t.dtype is torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def values_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def randn_bf16(shape, std=1.0, seed=0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).bfloat16().to(device)
