"""CPU oracle for the quantize + scaled-GEMM hot path.  TEST INFRASTRUCTURE ONLY.

A numpy restatement of the arithmetic of gau-nernst/quantized-training's hot path, written from
the reference's source (each function cites the file:line it follows). It exists to CHECK the
CUDA kernels: only the test-suite, the smoke entry and the benchmark's CPU-baseline leg may import
it. The product (the `gn_kernels`, `subclasses` and `other_optim` packages) never does.

Pinning: the reference ships no golden vectors for this path (its only checks are the inline
`assert_close` calls of benchmark_mm.py:98-121), so this oracle is pinned against outputs of the
reference's own Python functions run on CPU; `tests/golden/make_golden.py` generated those
fixtures by importing the reference, and `tests/test_oracle_golden.py` replays them.

All floating point here is IEEE fp32 via numpy (division and rint are correctly rounded /
half-to-even), bf16 is emulated on the fp32 bit pattern.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------------------------
# bf16 / fp8 emulation
# --------------------------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 (round-to-nearest-even); returns the 16-bit patterns as uint16."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = (bits + 0x7FFF + lsb) >> 16
    out = rounded.astype(np.uint32)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, (bits >> 16).astype(np.uint32) | 0x40, out)
    return out.astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to the nearest bf16, returned as fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round an fp32 array to `dtype` ('bf16' | 'f32'), returned as fp32 values."""
    if dtype == "bf16":
        return round_to_bf16(x)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(dtype)


def _e4m3_table() -> np.ndarray:
    """All 256 e4m3fn bit patterns decoded to fp32 (0x7F / 0xFF are NaN)."""
    vals = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            vals[b] = np.nan
        elif e == 0:
            vals[b] = s * (m / 8.0) * 2.0 ** (-6)
        else:
            vals[b] = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return vals


E4M3_VALUES = _e4m3_table()


def f32_to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e4m3fn bit patterns, round-to-nearest-even, saturating at +-448."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    # non-negative finite e4m3 values, ascending, codes 0..0x7E
    grid = E4M3_VALUES[:0x7F].astype(np.float64)
    hi = np.searchsorted(grid, a, side="left").clip(0, 0x7E)
    lo = (hi - 1).clip(0, 0x7E)
    d_hi = np.abs(grid[hi] - a)
    d_lo = np.abs(a - grid[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    codes = np.where(pick_lo, lo, hi).astype(np.uint8)
    return np.where(sign, codes | 0x80, codes).astype(np.uint8)


def e4m3_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[np.asarray(bits, dtype=np.uint8)]


def _e5m2_table() -> np.ndarray:
    """All 256 float8_e5m2 bit patterns decoded to fp32 (IEEE-like: exponent 31 is inf / NaN)."""
    vals = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 2) & 0x1F
        m = b & 0x3
        if e == 0x1F:
            vals[b] = s * np.inf if m == 0 else np.nan
        elif e == 0:
            vals[b] = s * (m / 4.0) * 2.0 ** (-14)
        else:
            vals[b] = s * (1.0 + m / 4.0) * 2.0 ** (e - 15)
    return vals


E5M2_VALUES = _e5m2_table()


def f32_to_e5m2_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e5m2 bit patterns, round-to-nearest-even, saturating at +-57344 (the other FP8
    format scaled_mm accepts, kernels/gn_kernels/triton_mm.py:359-361; its absmax constant is
    DTYPE_AMAX_LUT, kernels/gn_kernels/utils.py:7-11)."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x).astype(np.float64), 57344.0)
    grid = E5M2_VALUES[:0x7C].astype(np.float64)   # non-negative finite values, codes 0..0x7B
    hi = np.searchsorted(grid, a, side="left").clip(0, 0x7B)
    lo = (hi - 1).clip(0, 0x7B)
    d_hi = np.abs(grid[hi] - a)
    d_lo = np.abs(a - grid[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    codes = np.where(pick_lo, lo, hi).astype(np.uint8)
    return np.where(sign, codes | 0x80, codes).astype(np.uint8)


def e5m2_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return E5M2_VALUES[np.asarray(bits, dtype=np.uint8)]


# --------------------------------------------------------------------------------------------
# Philox4x32-10 (the stream the CUDA kernels draw stochastic-rounding uniforms from)
# --------------------------------------------------------------------------------------------

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, offset: int, seed: int) -> np.ndarray:
    """Philox4x32-10 (Salmon et al. 2011). counter: uint64 array; returns uint32 [..., 4].

    128-bit counter = (lo32(counter), hi32(counter), lo32(offset), hi32(offset)); key = seed.
    """
    counter = np.asarray(counter, dtype=np.uint64)
    c0 = counter & _MASK32
    c1 = counter >> np.uint64(32)
    c2 = np.full_like(c0, offset & 0xFFFFFFFF)
    c3 = np.full_like(c0, (offset >> 32) & 0xFFFFFFFF)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = (p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)
        n1 = p1 & _MASK32
        n2 = (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)
        n3 = p0 & _MASK32
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def philox_uniforms(n: int, seed: int, offset: int) -> np.ndarray:
    """The quantize kernels' stochastic-rounding uniforms: element i takes 16 bits of the stream --
    counter i // 8, word (i % 8) // 2, low half for even i, high half for odd i -- as
    u = bits * 2^-16 in [0, 1)."""
    n_ctr = (n + 7) // 8
    words = philox4x32_10(np.arange(n_ctr, dtype=np.uint64), offset, seed).reshape(-1)
    halves = np.stack([words & np.uint32(0xFFFF), words >> np.uint32(16)], axis=-1).reshape(-1)[:n]
    return (halves.astype(np.float32) * np.float32(1.0 / 65536.0)).astype(np.float32)


# --------------------------------------------------------------------------------------------
# quantize (subclasses/int8.py:12-26)
# --------------------------------------------------------------------------------------------

QMAX = {"int8": 127.0, "e4m3": 448.0, "e5m2": 57344.0}


def quantize_absmax(x: np.ndarray, *, axis: int = -1, eps: float = 1e-12, out: str = "int8",
                    scale_dtype: str = "bf16", uniforms: np.ndarray | None = None):
    """Symmetric absmax quantize along `axis` of a 2-D fp32 array (values of the input dtype).

    Follows quantize_int8, subclasses/int8.py:12-26, line by line:
      :15  scale = amax(|x|, dim, keepdim) / 127          (fp32)
      :17  x = x / scale.clip(eps)                        (fp32 IEEE division)
      :19-22  floor(x + u) when stochastic, else round() (half to even)
      :25  clip(-128, 127) -> int8
      :26  the returned scale is the unclamped one, cast to the input dtype
    `out='e4m3'` swaps 127 for 448 and the integer rounding for an e4m3 cast (the FP8 constant is
    DTYPE_AMAX_LUT, kernels/gn_kernels/utils.py:7-11). `uniforms` (same shape as x) selects
    stochastic rounding. Returns (q, scale_rounded_as_fp32) with q int8 or uint8 e4m3 bit patterns.
    """
    x = np.asarray(x, dtype=np.float32)
    qmax = np.float32(QMAX[out])
    scale = (np.abs(x).max(axis=axis, keepdims=True) / qmax).astype(np.float32)
    v = (x / np.maximum(scale, np.float32(eps))).astype(np.float32)
    if out == "int8":
        if uniforms is not None:
            v = np.floor((v + np.asarray(uniforms, dtype=np.float32)).astype(np.float32))
        else:
            v = np.rint(v)
        q = np.clip(v, -128, 127).astype(np.int8)
    else:
        if uniforms is not None:
            raise ValueError("stochastic rounding is defined for int8 only")
        q = f32_to_e4m3_bits(v) if out == "e4m3" else f32_to_e5m2_bits(v)
    return q, round_to(scale, scale_dtype)


def quantize_rowwise(x, **kw):
    """quantize_int8(x, dim=1): per-row scale [R,1]."""
    return quantize_absmax(x, axis=1, **kw)


def quantize_colwise_t(x, **kw):
    """quantize_int8(x.T, dim=1) then .contiguous(): returns (q [C,R], scale [C,1])
    (the B operand of _dynamic_int8_mm, subclasses/mixed_precision.py:102-105). Stochastic uniforms,
    if given, are indexed like the transposed tensor ([C,R])."""
    q, s = quantize_absmax(np.ascontiguousarray(np.asarray(x, dtype=np.float32).T), axis=1, **kw)
    return q, s


def quantize_tile(x: np.ndarray, tile: tuple[int, int], *, eps: float = 1e-12, out: str = "int8", scale_dtype: str = "bf16"):
    """quantize_int8's arithmetic applied per (tr x tc) tile; scale [ceil(R/tr), ceil(C/tc)]."""
    x = np.asarray(x, dtype=np.float32)
    R, C = x.shape
    tr, tc = tile
    nr, nc = -(-R // tr), -(-C // tc)
    pad = np.zeros((nr * tr, nc * tc), dtype=np.float32)
    pad[:R, :C] = x
    t = pad.reshape(nr, tr, nc, tc)
    qmax = np.float32(QMAX[out])
    scale = (np.abs(t).max(axis=(1, 3)) / qmax).astype(np.float32)
    v = (t / np.maximum(scale, np.float32(eps))[:, None, :, None]).astype(np.float32).reshape(nr * tr, nc * tc)[:R, :C]
    q = np.clip(np.rint(v), -128, 127).astype(np.int8) if out == "int8" else (f32_to_e4m3_bits(v) if out == "e4m3" else f32_to_e5m2_bits(v))
    return q, round_to(scale, scale_dtype)


# --------------------------------------------------------------------------------------------
# GEMMs (kernels/gn_kernels/triton_mm.py)
# --------------------------------------------------------------------------------------------


def int8_mm(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """int32 C = A @ B, exact (int8_mm, triton_mm.py:112-128; pinned to torch._int_mm by
    benchmark_mm.py:112). float64 BLAS is exact here: |sum| <= 128*128*K < 2^53."""
    acc = np.asarray(A, dtype=np.float64) @ np.asarray(B, dtype=np.float64)
    return acc.astype(np.int64).astype(np.int32)


def _decode(a: np.ndarray, kind: str) -> np.ndarray:
    """Operand values as float64. kind: 'int8', 'e4m3', 'e5m2', or a pair 'e4m3/e5m2' (A / B formats)."""
    if kind == "int8":
        return np.asarray(a, dtype=np.float64)
    if kind == "e4m3":
        return e4m3_bits_to_f32(a).astype(np.float64)
    if kind == "e5m2":
        return e5m2_bits_to_f32(a).astype(np.float64)
    raise ValueError(kind)


def _kinds(kind: str) -> tuple[str, str]:
    return tuple(kind.split("/")) if "/" in kind else (kind, kind)


def scaled_mm(A, B, scale_a, scale_b, *, kind: str = "int8", out_dtype: str = "bf16") -> np.ndarray:
    """Row/column-scaled GEMM epilogue of _scaled_mm_kernel (triton_mm.py:210-216):
    fp32(acc) * row_scale * col_scale evaluated left to right in fp32, then cast to the scale dtype
    (:386). For int8 the accumulator is the exact int32; for fp8 it is the fp32-rounded exact sum
    (tensor cores may differ in the last bits, hence a tolerance in the fp8 tests).
    scale_a [M,1], scale_b [1,N] or [1,1], given as fp32 values of the scale dtype."""
    ka, kb_ = _kinds(kind)
    acc = _decode(A, ka) @ _decode(B, kb_)
    acc32 = acc.astype(np.float32)
    sa = np.asarray(scale_a, dtype=np.float32).reshape(-1, 1)
    sb = np.asarray(scale_b, dtype=np.float32).reshape(1, -1)
    out = ((acc32 * sa).astype(np.float32) * sb).astype(np.float32)
    return round_to(out, out_dtype)


def tile_scaled_mm(A, B, scale_a, scale_b, *, kind: str = "int8", out_dtype: str = "bf16") -> np.ndarray:
    """_tile_scaled_mm_kernel (triton_mm.py:314-331): per K-block kb,
    acc += fp32(A_kb @ B_kb) * a_scale[m/QM, kb] * b_scale[kb, n/QN], fp32, blocks in order."""
    A, B = np.asarray(A), np.asarray(B)
    M, K = A.shape
    N = B.shape[1]
    sa = np.asarray(scale_a, dtype=np.float32)
    sb = np.asarray(scale_b, dtype=np.float32)
    qm, qk, qn = M // sa.shape[0], K // sa.shape[1], N // sb.shape[1]
    ka, kb_ = _kinds(kind)
    Ad, Bd = _decode(A, ka), _decode(B, kb_)
    acc = np.zeros((M, N), dtype=np.float32)
    rows = np.arange(M) // qm
    cols = np.arange(N) // qn
    for kb in range(K // qk):
        part = (Ad[:, kb * qk:(kb + 1) * qk] @ Bd[kb * qk:(kb + 1) * qk, :]).astype(np.float32)
        part = (part * sa[rows, kb][:, None]).astype(np.float32)
        part = (part * sb[kb, cols][None, :]).astype(np.float32)
        acc = (acc + part).astype(np.float32)
    return round_to(acc, out_dtype)


def dynamic_int8_mm(A: np.ndarray, B: np.ndarray, *, dtype: str = "bf16", uniforms_a=None, uniforms_bt=None) -> np.ndarray:
    """_dynamic_int8_mm (subclasses/mixed_precision.py:100-108): quantize A per row, B per column
    (as rows of B.T), then scaled_mm. A [M,K], B [K,N] hold values of `dtype`."""
    qa, sa = quantize_rowwise(A, scale_dtype=dtype, uniforms=uniforms_a)
    qbt, sb = quantize_colwise_t(B, scale_dtype=dtype, uniforms=uniforms_bt)
    return scaled_mm(qa, qbt.T, sa, sb.T, out_dtype=dtype)


# --------------------------------------------------------------------------------------------
# INT8 mixed-precision linear (subclasses/mixed_precision.py:146-193)
# --------------------------------------------------------------------------------------------


def mixed_precision_linear_forward(x: np.ndarray, w: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """forward, mixed_precision.py:147-158 with config.output: x [M,K] @ w[N,K].T via dynamic int8."""
    return dynamic_int8_mm(x, np.asarray(w, dtype=np.float32).T, dtype=dtype)


def mixed_precision_linear_backward(x, w, gy, dtype: str = "bf16"):
    """backward, mixed_precision.py:167-193 with config.grad_input and config.grad_weight:
    grad_input = dyn_mm(gy, w) (:176-181); grad_weight = dyn_mm(x.T, gy).T (:183-188)."""
    x, w, gy = (np.asarray(t, dtype=np.float32) for t in (x, w, gy))
    grad_input = dynamic_int8_mm(gy, w, dtype=dtype)
    grad_weight = dynamic_int8_mm(np.ascontiguousarray(x.T), gy, dtype=dtype).T
    return grad_input, grad_weight


# --------------------------------------------------------------------------------------------
# BitNet b1.58 helpers (subclasses/bitnet.py)
# --------------------------------------------------------------------------------------------


def bitnet_scale(w: np.ndarray) -> np.float32:
    """get_bitnet_scale, bitnet.py:110-112: fp32 mean of |w|. Summation order is unspecified in the
    reference (a torch reduction); float64 accumulation here, compared with a tolerance."""
    return np.float32(np.abs(np.asarray(w, dtype=np.float32)).astype(np.float64).mean())


def bitnet_quantize_weight(w: np.ndarray, scale, eps: float = 1e-5) -> np.ndarray:
    """quantize_bitnet_weight, bitnet.py:115-118: round(w / clip(scale, eps)) clipped to [-1, 1]."""
    v = (np.asarray(w, dtype=np.float32) / np.maximum(np.float32(scale), np.float32(eps))).astype(np.float32)
    return np.clip(np.rint(v), -1, 1).astype(np.int8)


def pack_i2(x: np.ndarray) -> np.ndarray:
    """_pack_i2_in_i8, bitnet.py:185-195: four 2-bit two's-complement values per byte, first value
    in the top bits."""
    u = np.asarray(x, dtype=np.int8).view(np.uint8).astype(np.uint32) & 0x3
    return ((u[:, 0::4] << 6) | (u[:, 1::4] << 4) | (u[:, 2::4] << 2) | u[:, 3::4]).astype(np.uint8).view(np.int8)


def unpack_i2(p: np.ndarray) -> np.ndarray:
    """_unpack_i2_in_i8, bitnet.py:198-201: sign-extending inverse of pack_i2."""
    u = np.asarray(p, dtype=np.int8).view(np.uint8).astype(np.int32)
    fields = np.stack([(u >> 6) & 3, (u >> 4) & 3, (u >> 2) & 3, u & 3], axis=-1)
    fields = np.where(fields >= 2, fields - 4, fields)
    return fields.reshape(p.shape[0], -1).astype(np.int8)


# --------------------------------------------------------------------------------------------
# AdamW with bf16 stochastic rounding (other_optim/bf16_sr.py:78-124)
# --------------------------------------------------------------------------------------------


def adamw_bf16_sr(p, grad, step: float, exp_avg, exp_avg_sq, lr: float, beta1: float, beta2: float, weight_decay: float,
                  eps: float, rand16: np.ndarray | None):
    """One `adamw` step, bf16_sr.py:78-124. p/grad/exp_avg/exp_avg_sq: fp32 arrays holding bf16
    values. rand16: uint32 array of 16-bit randoms (the `random_() & 0xFFFF` of :113-114) or None
    for a plain round-to-nearest write-back. Returns (new_p, new_exp_avg, new_exp_avg_sq) as fp32
    arrays of bf16 values.

      :91-92   bias corrections 1 - beta**step
      :96-97   lerp(exp_avg, grad, 1-beta1), lerp(exp_avg_sq, grad^2, 1-beta2)   (fp32)
      :99-100  states written back in bf16
      :102-106 denom = sqrt(v)/sqrt(bc2) + eps ; new_p = p - lr*wd*p - lr*(m/bc1)/denom
      :108-122 bits(new_p) + rand16, low 16 bits cleared
    """
    f = np.float32
    p, grad, m, v = (np.asarray(t, dtype=np.float32) for t in (p, grad, exp_avg, exp_avg_sq))
    bc1 = f(1.0) - f(beta1) ** f(step)
    bc2 = f(1.0) - f(beta2) ** f(step)
    w1, w2 = f(1.0 - beta1), f(1.0 - beta2)
    new_m = lerp(m, grad, w1)
    new_v = lerp(v, (grad * grad).astype(np.float32), w2)
    denom = (np.sqrt(new_v).astype(np.float32) / np.sqrt(bc2).astype(np.float32) + f(eps)).astype(np.float32)
    numer = (new_m / bc1).astype(np.float32)
    lr = f(lr)
    new_p = (p - (lr * f(weight_decay)) * p).astype(np.float32)
    new_p = (new_p - ((lr * numer).astype(np.float32) / denom).astype(np.float32)).astype(np.float32)
    if rand16 is not None:
        bits = new_p.view(np.uint32).astype(np.uint64) + (np.asarray(rand16, dtype=np.uint64) & 0xFFFF)
        bits = (bits & 0xFFFFFFFF).astype(np.uint32) & np.uint32(0xFFFF0000)
        out_p = bits.view(np.float32)
    else:
        out_p = round_to_bf16(new_p)
    return out_p, round_to_bf16(new_m), round_to_bf16(new_v)


def fma32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Correctly rounded fp32 fused multiply-add a*b + c, computed through float64.

    The product of two fp32 values is exact in float64; the float64 sum is rounded once, and the
    rare double-rounding case (the float64 sum lands exactly on an fp32 tie while the discarded
    error is non-zero) is repaired with the exact TwoSum error term."""
    a64, b64, c64 = (np.asarray(t, dtype=np.float32).astype(np.float64) for t in (a, b, c))
    prod = a64 * b64
    s = prod + c64
    bb = s - prod
    err = (prod - (s - bb)) + (c64 - bb)
    r = s.astype(np.float32)
    d = s - r.astype(np.float64)
    up = np.nextafter(r, np.float32(np.inf)).astype(np.float64)
    dn = np.nextafter(r, np.float32(-np.inf)).astype(np.float64)
    with np.errstate(invalid="ignore"):
        tie_up = (d > 0) & (d == (up - r.astype(np.float64)) / 2) & (err > 0)
        tie_dn = (d < 0) & (d == (dn - r.astype(np.float64)) / 2) & (err < 0)
    r = np.where(tie_up, up.astype(np.float32), r)
    r = np.where(tie_dn, dn.astype(np.float32), r)
    return r.astype(np.float32)


def lerp(a: np.ndarray, b: np.ndarray, w: np.float32) -> np.ndarray:
    """torch.lerp with a scalar weight: ATen evaluates `a + w * (b - a)` for |w| < 0.5 as one fused
    multiply-add (vectorised fmadd on CPU, contracted FFMA on CUDA), else `b - (b - a) * (1 - w)`
    the same way."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    diff = (b - a).astype(np.float32)
    if abs(w) < 0.5:
        return fma32(np.full_like(diff, w), diff, a)
    return fma32(-diff, np.full_like(diff, np.float32(1) - w), b)
