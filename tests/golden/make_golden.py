"""Generates the golden fixtures in this folder by running the REFERENCE project's own Python
functions on CPU. Needs the reference checkout; the fixtures it writes are what travels.

    python tests/golden/make_golden.py /path/to/quantized-training

What is recorded (all small, seeded, CPU):
  quantize_*.npz     quantize_int8 (subclasses/int8.py:12-26): round-to-nearest and stochastic
                     (the uniforms torch.rand_like drew are captured by re-seeding)
  scaled_mm_ref.npz  scaled_mm_ref (benchmark_mm.py:46-50) on row/col and tile scales, the function
                     the reference checks its kernels against with atol/rtol (benchmark_mm.py:113-121)
  mp_linear.npz      forward + backward of a Linear converted by convert_mixed_precision
                     (subclasses/mixed_precision.py:146-205); gn_kernels::scaled_mm is given a CPU
                     implementation made of torch._int_mm plus the Triton epilogue's arithmetic
                     (kernels/gn_kernels/triton_mm.py:210-216), the ops having no CPU kernel
  adamw_bf16_sr.npz  other_optim/bf16_sr.py:78-124 `adamw`, eager, with and without stochastic rounding
  bitnet.npz         get_bitnet_scale / quantize_bitnet_weight / pack / unpack (subclasses/bitnet.py)
  config1_digest.json  SHA-256 digests of the 1024^2, seed-2024 configuration's tensors
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().contiguous().numpy().copy()


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "kernels"))
    sys.path.insert(0, ref_root)
    import gn_kernels  # noqa: F401  (registers the op schemas)
    from gn_kernels._lib import lib
    import subclasses
    from subclasses.int8 import quantize_int8, Int8LinearWeight
    from subclasses.bitnet import get_bitnet_scale, quantize_bitnet_weight, _pack_i2_in_i8, _unpack_i2_in_i8
    from subclasses.mixed_precision import MixedPrecisionConfig, convert_mixed_precision, _dynamic_int8_mm
    from other_optim.bf16_sr import adamw
    import benchmark_mm

    # CPU stand-in for the CUDA-only op: exact int32 accumulate, then the Triton kernel's epilogue
    @torch.library.impl(lib, "scaled_mm", "CPU")
    def _(A, B, row_scale, col_scale):
        acc = torch._int_mm(A.contiguous(), B.contiguous()) if A.shape[0] > 16 else (A.int() @ B.int())
        return (acc.float() * row_scale.float() * col_scale.float()).to(row_scale.dtype)

    # ---------------- quantize_int8 ----------------
    cases = {}
    torch.manual_seed(1234)
    specs = [
        ("bf16_64x96", (64, 96), torch.bfloat16, 1.0, 1e-12),
        ("bf16_33x257", (33, 257), torch.bfloat16, 1.0, 1e-12),
        ("bf16_128x1000_small", (128, 1000), torch.bfloat16, 0.02, 1e-12),
        ("bf16_16x2048_eps1e-5", (16, 2048), torch.bfloat16, 1e-4, 1e-5),
        ("f32_40x72", (40, 72), torch.float32, 3.0, 1e-12),
        ("bf16_7x5000", (7, 5000), torch.bfloat16, 1.0, 1e-12),
    ]
    for name, shape, dtype, std, eps in specs:
        x = (torch.randn(shape) * std).to(dtype)
        x[1] = 0  # an all-zero row exercises the eps clamp
        x[2, 3] = float(x.abs().max()) * 4  # an outlier
        for dim in (1, 0):
            q, s = quantize_int8(x, dim=dim, eps=eps)
            cases[f"{name}_dim{dim}_x"] = bf16_bits(x) if dtype is torch.bfloat16 else f32(x)
            cases[f"{name}_dim{dim}_q"] = q.numpy()
            cases[f"{name}_dim{dim}_scale"] = bf16_bits(s) if dtype is torch.bfloat16 else f32(s)
            cases[f"{name}_dim{dim}_eps"] = np.float64(eps)
        # stochastic: capture the uniforms by re-seeding
        torch.manual_seed(99)
        u = torch.rand_like(x.float())
        torch.manual_seed(99)
        q, s = quantize_int8(x, True, dim=1, eps=eps)
        cases[f"{name}_sr_u"] = u.numpy()
        cases[f"{name}_sr_q"] = q.numpy()
    np.savez_compressed(HERE / "quantize.npz", **cases)

    # ---------------- scaled_mm_ref ----------------
    torch.manual_seed(2025 * 2024)
    M, N, K = 256, 384, 512
    A = torch.randint(-128, 127, (M, K), dtype=torch.int8)
    B = torch.randint(-128, 127, (K, N), dtype=torch.int8)
    sA = torch.randn(M, 1).div(128).bfloat16()
    sB = torch.randn(1, N).div(128).bfloat16()
    tsA = torch.randn(M, K // 128).div(128).bfloat16()
    tsB = torch.randn(K // 128, N // 128).div(128).bfloat16()
    A8 = torch.randn(M, K).to(torch.float8_e4m3fn)
    B8 = torch.randn(K, N).to(torch.float8_e4m3fn)
    out = dict(
        A=A.numpy(), B=B.numpy(), sA=bf16_bits(sA), sB=bf16_bits(sB), tsA=bf16_bits(tsA), tsB=bf16_bits(tsB),
        int_mm=torch._int_mm(A, B).numpy(),
        rowcol=bf16_bits(benchmark_mm.scaled_mm_ref(A, B, sA, sB)),
        tile=bf16_bits(benchmark_mm.scaled_mm_ref(A, B, tsA, tsB)),
        A8=A8.view(torch.uint8).numpy(), B8=B8.view(torch.uint8).numpy(),
        f8_rowcol=bf16_bits(benchmark_mm.scaled_mm_ref(A8, B8, sA, sB)),
        f8_tile=bf16_bits(benchmark_mm.scaled_mm_ref(A8, B8, tsA, tsB)),
        f8_plain=bf16_bits((A8.float() @ B8.float()).bfloat16()),
    )
    np.savez_compressed(HERE / "scaled_mm_ref.npz", **out)

    # ---------------- mixed-precision linear fwd/bwd ----------------
    torch.manual_seed(7)
    lin = torch.nn.Linear(192, 160, bias=True).bfloat16()
    w0 = lin.weight.detach().clone()
    b0 = lin.bias.detach().clone()
    convert_mixed_precision(lin, config=MixedPrecisionConfig())
    x = torch.randn(3, 40, 192).bfloat16().requires_grad_()
    y = lin(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    dyn = _dynamic_int8_mm(x.detach().view(-1, 192), w0.T, False)
    np.savez_compressed(
        HERE / "mp_linear.npz",
        x=bf16_bits(x), w=bf16_bits(w0), b=bf16_bits(b0), gy=bf16_bits(gy), y=bf16_bits(y),
        gx=bf16_bits(x.grad), gw=bf16_bits(lin.weight.grad), gb=bf16_bits(lin.bias.grad), dyn=bf16_bits(dyn),
    )

    # ---------------- AdamW bf16 SR ----------------
    torch.manual_seed(11)
    n = 4096
    rec = {}
    for tag, sr in (("sr", True), ("rn", False)):
        p = torch.randn(n).bfloat16()
        g = (torch.randn(n) * 0.1).bfloat16()
        m = (torch.randn(n) * 0.01).bfloat16()
        v = (torch.rand(n) * 1e-3).bfloat16()
        rec[f"{tag}_p"], rec[f"{tag}_g"], rec[f"{tag}_m"], rec[f"{tag}_v"] = (bf16_bits(t) for t in (p, g, m, v))
        step = torch.tensor(3.0)
        lr = torch.tensor(1e-3)
        torch.manual_seed(5)
        rand = torch.empty(n, dtype=torch.int32).random_() & 0xFFFF
        torch.manual_seed(5)
        p_run = p.clone() if sr else p.float()  # SR only applies to bf16 params
        adamw(p_run, g, step, m, v, lr, 0.9, 0.999, 0.01, 1e-8, sr)
        rec[f"{tag}_rand"] = rand.numpy().astype(np.uint32)
        rec[f"{tag}_p_out"] = bf16_bits(p_run) if sr else f32(p_run)
        rec[f"{tag}_m_out"], rec[f"{tag}_v_out"] = bf16_bits(m), bf16_bits(v)
    rec["hyper"] = np.array([3.0, 1e-3, 0.9, 0.999, 0.01, 1e-8], dtype=np.float64)
    np.savez_compressed(HERE / "adamw_bf16_sr.npz", **rec)

    # ---------------- BitNet ----------------
    torch.manual_seed(21)
    w = (torch.randn(48, 64) * 0.05).bfloat16()
    sc = get_bitnet_scale(w)
    wq = quantize_bitnet_weight(w, sc)
    packed = _pack_i2_in_i8(wq)
    np.savez_compressed(
        HERE / "bitnet.npz", w=bf16_bits(w), scale=np.float32(sc.item()), wq=wq.numpy(), packed=packed.numpy(),
        unpacked=_unpack_i2_in_i8(packed).numpy(),
    )

    # ---------------- Int8LinearWeight ----------------
    torch.manual_seed(31)
    w = torch.randn(24, 40).bfloat16()
    qw = Int8LinearWeight.from_float(w)
    np.savez_compressed(HERE / "int8_weight.npz", w=bf16_bits(w), int_data=qw.int_data.numpy(), scale=bf16_bits(qw.scale),
                        deq=bf16_bits(qw.dequantize()))

    # ---------------- digests of the 1024^2, seed-2024 configuration ----------------
    torch.manual_seed(2024)
    A = torch.randn(1024, 1024).bfloat16()
    B = (torch.randn(1024, 1024) * 0.02).bfloat16()
    qa, sa = quantize_int8(A, dim=1)
    qb, sb = quantize_int8(B, dim=1)
    acc = torch._int_mm(qa, qb.T.contiguous())
    outp = (acc.float() * sa.float() * sb.float().T).bfloat16()

    def dig(a: np.ndarray) -> str:
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()

    digest = dict(
        A=dig(bf16_bits(A)), B=dig(bf16_bits(B)), qa=dig(qa.numpy()), qb=dig(qb.numpy()), sa=dig(bf16_bits(sa)),
        sb=dig(bf16_bits(sb)), acc=dig(acc.numpy()), out=dig(bf16_bits(outp)),
        qa_range=[int(qa.min()), int(qa.max())], acc_absmax=int(acc.abs().max()),
        torch_version=torch.__version__,
    )
    (HERE / "config1_digest.json").write_text(json.dumps(digest, indent=1) + "\n")
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of gau-nernst/quantized-training>")
    main(sys.argv[1])
