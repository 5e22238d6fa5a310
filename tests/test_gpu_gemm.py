"""GPU parity of the tcgen05 GEMMs: exact int32 accumulators, bit-exact scaled bf16 outputs for
int8 (the epilogue is deterministic fp32), reference tolerances for fp8 and tile-scaled variants."""
import numpy as np
import pytest
import torch

from oracle import reference_math as om
from tests.helpers import bits_of, randn_bf16, values_of

pytestmark = pytest.mark.gpu

import gn_kernels  # noqa: E402
from gn_kernels import _native as nv  # noqa: E402

LAYOUTS = ["A@B.T", "A@B", "A.T@B", "A.T@B.T"]


@pytest.fixture(params=[0, 1, 2], ids=["cg_auto", "cg1", "cg2"])
def cta_group(request):
    """Run a test with the GEMM's CTA-pair mode chosen automatically, forced off and forced on."""
    nv.check(nv.load().qt_set_gemm_cta_group(request.param))
    yield request.param
    nv.check(nv.load().qt_set_gemm_cta_group(0))


def to_layout(A, B, name):
    """A [M,K], B [K,N] re-laid-out like the reference benchmark's --a/b_column_major flags
    (benchmark_mm.py:33-34,91-96)."""
    a = A.T.contiguous().T if name.startswith("A.T") else A.contiguous()
    b = B.T.contiguous().T if name.endswith("B.T") else B.contiguous()
    return a, b


def rand_i8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-128, 127, shape, dtype=torch.int8, generator=g).cuda()


@pytest.mark.parametrize("mnk", [(128, 256, 128), (128, 256, 640), (256, 512, 256), (1024, 1024, 1024), (300, 520, 272),
                                 (100, 72, 48), (1, 16, 16), (130, 8, 4096), (2048, 32, 64), (17, 1000, 336)])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_int8_mm_exact(mnk, layout, cta_group):
    M, N, K = mnk
    A, B = rand_i8((M, K), 1 + M), rand_i8((K, N), 2 + N)
    A[0, :] = -128
    B[:, 0] = -128  # the extreme products
    a, b = to_layout(A, B, layout)
    out = gn_kernels.int8_mm(a, b)
    want = om.int8_mm(A.cpu().numpy(), B.cpu().numpy())
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    assert nv.device_status() == 0


def test_int8_mm_odd_shapes_are_padded_by_the_wrapper():
    for (M, N, K) in [(33, 45, 50), (7, 9, 13), (64, 64, 100)]:
        A, B = rand_i8((M, K), 5), rand_i8((K, N), 6)
        out = gn_kernels.int8_mm(A, B)
        np.testing.assert_array_equal(out.cpu().numpy(), om.int8_mm(A.cpu().numpy(), B.cpu().numpy()))
        out = gn_kernels.int8_mm(A[:, ::1], B.T.contiguous().T)
        np.testing.assert_array_equal(out.cpu().numpy(), om.int8_mm(A.cpu().numpy(), B.cpu().numpy()))


def test_int8_mm_matches_reference_fixture(golden_dir):
    g = np.load(golden_dir / "scaled_mm_ref.npz")
    A, B = torch.from_numpy(g["A"]).cuda(), torch.from_numpy(g["B"]).cuda()
    np.testing.assert_array_equal(gn_kernels.int8_mm(A, B).cpu().numpy(), g["int_mm"])


def test_degenerate_sizes():
    A = torch.zeros((0, 64), dtype=torch.int8, device="cuda")
    B = torch.zeros((64, 32), dtype=torch.int8, device="cuda")
    assert gn_kernels.int8_mm(A, B).shape == (0, 32)
    A = torch.zeros((16, 0), dtype=torch.int8, device="cuda")
    B = torch.zeros((0, 32), dtype=torch.int8, device="cuda")
    out = gn_kernels.int8_mm(A, B)
    assert out.shape == (16, 32) and int(out.abs().sum()) == 0


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("mnk", [(1024, 1024, 1024), (300, 520, 272), (128, 264, 128)])
def test_scaled_mm_int8_bit_exact(mnk, layout, cta_group):
    M, N, K = mnk
    A, B = rand_i8((M, K), 11), rand_i8((K, N), 12)
    g = torch.Generator().manual_seed(13)
    sa = (torch.randn(M, 1, generator=g) / 128).bfloat16().cuda()
    sb = (torch.randn(1, N, generator=g) / 128).bfloat16().cuda()
    a, b = to_layout(A, B, layout)
    out = gn_kernels.scaled_mm(a, b, sa, sb)
    want = om.scaled_mm(A.cpu().numpy(), B.cpu().numpy(), values_of(sa), values_of(sb))
    np.testing.assert_array_equal(values_of(out), want)
    assert out.dtype is torch.bfloat16
    # fp32 scales -> fp32 output (scale dtype decides, triton_mm.py:386)
    out32 = gn_kernels.scaled_mm(a, b, sa.float(), sb.float())
    want32 = om.scaled_mm(A.cpu().numpy(), B.cpu().numpy(), values_of(sa), values_of(sb), out_dtype="f32")
    np.testing.assert_array_equal(out32.cpu().numpy(), want32)


def test_scaled_mm_scalar_and_column_vector_scales():
    M, N, K = 256, 384, 512
    A, B = rand_i8((M, K), 21), rand_i8((K, N), 22)
    sa = (torch.rand(M, 1) / 64).bfloat16().cuda()
    one = torch.tensor(0.0123).bfloat16().cuda()
    want = om.scaled_mm(A.cpu().numpy(), B.cpu().numpy(), values_of(sa), values_of(one).reshape(1, 1))
    np.testing.assert_array_equal(values_of(gn_kernels.scaled_mm(A, B, sa, one.view(1, 1))), want)
    np.testing.assert_array_equal(values_of(gn_kernels.scaled_mm(A, B, sa, one)), want)           # 0-dim (BitNet call site)
    sb_col = (torch.rand(N, 1) / 64).bfloat16().cuda()                                           # [N,1] (Int8LinearWeight.scale)
    want = om.scaled_mm(A.cpu().numpy(), B.cpu().numpy(), values_of(sa), values_of(sb_col).reshape(1, -1))
    np.testing.assert_array_equal(values_of(gn_kernels.scaled_mm(A, B, sa, sb_col)), want)


def test_scaled_mm_reference_fixture_and_tolerances(golden_dir):
    """Inputs drawn like benchmark_mm.py:78-89; acceptance as benchmark_mm.py:113-118."""
    g = np.load(golden_dir / "scaled_mm_ref.npz")
    A, B = torch.from_numpy(g["A"]).cuda(), torch.from_numpy(g["B"]).cuda()
    sA = torch.from_numpy(g["sA"].view(np.int16).copy()).view(torch.bfloat16).cuda()
    sB = torch.from_numpy(g["sB"].view(np.int16).copy()).view(torch.bfloat16).cuda()
    out = gn_kernels.scaled_mm(A, B, sA, sB)
    np.testing.assert_allclose(values_of(out), om.bf16_bits_to_f32(g["rowcol"]), atol=4e-4, rtol=1e-2)


def test_config1_dynamic_quantize_plus_gemm(golden_dir):
    """The reference's CPU-runnable configuration: A ~ N(0,1), B ~ N(0,0.02), 1024^2, seed 2024, A @ B.T row-wise INT8."""
    torch.manual_seed(2024)
    A = torch.randn(1024, 1024).bfloat16()
    B = (torch.randn(1024, 1024) * 0.02).bfloat16()
    qa, sa = gn_kernels.quantize_rowwise(A.cuda())
    qb, sb = gn_kernels.quantize_rowwise(B.cuda())
    acc = gn_kernels.int8_mm(qa, qb.T)
    out = gn_kernels.scaled_mm(qa, qb.T, sa, sb.T.contiguous())
    oqa, osa = om.quantize_rowwise(A.float().numpy())
    oqb, osb = om.quantize_rowwise(B.float().numpy())
    np.testing.assert_array_equal(qa.cpu().numpy(), oqa)
    np.testing.assert_array_equal(qb.cpu().numpy(), oqb)
    np.testing.assert_array_equal(acc.cpu().numpy(), om.int8_mm(oqa, oqb.T))
    np.testing.assert_array_equal(values_of(out), om.scaled_mm(oqa, oqb.T, osa, osb.T))
    assert int(qa.min()) >= -127 and int(qa.max()) <= 127


@pytest.mark.parametrize("layout", ["A@B.T", "A@B", "A.T@B"])
def test_scaled_mm_fp8(layout, cta_group):
    M, N, K = 512, 768, 1024
    g = torch.Generator().manual_seed(31)
    A8 = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn).cuda()
    B8 = torch.randn(K, N, generator=g).to(torch.float8_e4m3fn).cuda()
    sa = (torch.randn(M, 1, generator=g) / 128).bfloat16().cuda()
    sb = (torch.randn(1, N, generator=g) / 128).bfloat16().cuda()
    a, b = to_layout(A8, B8, layout)
    out = gn_kernels.scaled_mm(a, b, sa, sb)
    want = om.scaled_mm(bits_of(A8), bits_of(B8), values_of(sa), values_of(sb), kind="e4m3")
    # north-star tolerance for scaled bf16 outputs: 1e-2 relative (fp32 accumulation order differs)
    np.testing.assert_allclose(values_of(out), want, rtol=1e-2, atol=1e-4)


def test_full_size_gemm_properties():
    """8192^3 (the benchmark size): linearity in the row scale, agreement of the three layouts, and
    a sampled exact check of the int32 accumulators."""
    S = 8192
    A, B = rand_i8((S, S), 41), rand_i8((S, S), 42)
    sa = torch.full((S, 1), 2.0 ** -7, dtype=torch.bfloat16, device="cuda")
    sb = torch.full((1, S), 2.0 ** -6, dtype=torch.bfloat16, device="cuda")
    base = gn_kernels.scaled_mm(A, B.T.contiguous().T, sa, sb)
    acc = gn_kernels.int8_mm(A, B)
    assert torch.equal(base, (acc.float() * 2.0 ** -13).bfloat16())           # power-of-two scales are exact
    assert torch.equal(gn_kernels.scaled_mm(A, B, sa * 2, sb), (acc.float() * 2.0 ** -12).bfloat16())
    assert torch.equal(gn_kernels.int8_mm(A.T.contiguous().T, B), acc)
    rows = torch.tensor([0, 1, 4095, 8191], device="cuda")
    want = om.int8_mm(A[rows].cpu().numpy(), B.cpu().numpy())
    np.testing.assert_array_equal(acc[rows].cpu().numpy(), want)
    assert nv.device_status() == 0


@pytest.mark.parametrize("layout", ["A@B.T", "A@B", "A.T@B"])
@pytest.mark.parametrize("tiles", [(1, 128), (128, 128)])
def test_tile_scaled_mm_int8(layout, tiles):
    """DeepSeek-style 1x128 activation / 128x128 weight tiles (benchmark_mm.py:87-89), and 128x128 on
    both sides; acceptance as benchmark_mm.py:119-121 (atol 1e-4, rtol 1e-2) against the oracle."""
    M, N, K = 384, 512, 640
    qm = tiles[0]
    A, B = rand_i8((M, K), 51), rand_i8((K, N), 52)
    g = torch.Generator().manual_seed(53)
    sa = (torch.randn(M // qm, K // 128, generator=g) / 128).bfloat16().cuda()
    sb = (torch.randn(K // 128, N // 128, generator=g) / 128).bfloat16().cuda()
    a, b = to_layout(A, B, layout)
    out = gn_kernels.scaled_mm(a, b, sa, sb)
    want = om.tile_scaled_mm(A.cpu().numpy(), B.cpu().numpy(), values_of(sa), values_of(sb))
    np.testing.assert_allclose(values_of(out), want, atol=1e-4, rtol=1e-2)
    assert out.dtype is torch.bfloat16 and nv.device_status() == 0
    # column-major scale tensors (the benchmark re-lays them out with the operands) are read by stride
    out2 = gn_kernels.scaled_mm(a, b, sa.T.contiguous().T, sb.T.contiguous().T)
    assert torch.equal(out, out2)


def test_tile_scaled_mm_reference_fixture_and_fp8(golden_dir):
    g = np.load(golden_dir / "scaled_mm_ref.npz")

    def bf(a):
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).cuda()

    A, B = torch.from_numpy(g["A"]).cuda(), torch.from_numpy(g["B"]).cuda()
    out = gn_kernels.scaled_mm(A, B, bf(g["tsA"]), bf(g["tsB"]))
    np.testing.assert_allclose(values_of(out), om.bf16_bits_to_f32(g["tile"]), atol=1e-4, rtol=1e-2)
    A8 = torch.from_numpy(g["A8"]).cuda().view(torch.float8_e4m3fn)
    B8 = torch.from_numpy(g["B8"]).cuda().view(torch.float8_e4m3fn)
    out8 = gn_kernels.scaled_mm(A8, B8, bf(g["tsA"]), bf(g["tsB"]))
    np.testing.assert_allclose(values_of(out8), om.bf16_bits_to_f32(g["f8_tile"]), rtol=1.6e-2, atol=2e-5)


def test_tile_scaled_mm_rejects_unsupported_blocks():
    A, B = rand_i8((128, 256), 1), rand_i8((256, 128), 2)
    sa = torch.ones((128, 4), dtype=torch.bfloat16, device="cuda")   # qk = 64
    sb = torch.ones((4, 1), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="reduction block must be a multiple of 128"):
        gn_kernels.scaled_mm(A, B, sa, sb)
    sa = torch.ones((128, 2), dtype=torch.bfloat16, device="cuda")   # qk = 128, qn = 8
    sb = torch.ones((2, 16), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="qn one of 16, 32, 64"):
        gn_kernels.scaled_mm(A, B, sa, sb)


@pytest.mark.parametrize("blocks", [(1, 256, 128), (128, 256, 256), (1, 128, 64), (4, 128, 32), (1, 512, 16), (128, 128, 256)])
@pytest.mark.parametrize("kind", ["int8", "e4m3"])
def test_tile_scaled_mm_infers_other_block_shapes(blocks, kind):
    """The reference infers (QM, QK, QN) from the scale shapes (kernels/gn_kernels/triton_mm.py:419,434-437).
    Here: any QM, QK a multiple of 128, QN one of 16 / 32 / 64 or a multiple of 128."""
    qm, qk, qn = blocks
    M, N, K = 256, 512, 1024
    g = torch.Generator().manual_seed(qm + qk + qn)
    if kind == "int8":
        A, B = rand_i8((M, K), 61), rand_i8((K, N), 62)
    else:
        A = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn).cuda()
        B = torch.randn(K, N, generator=g).to(torch.float8_e4m3fn).cuda()
    sa = (torch.rand(M // qm, K // qk, generator=g) / 64 + 1e-3).bfloat16().cuda()
    sb = (torch.rand(K // qk, N // qn, generator=g) / 64 + 1e-3).bfloat16().cuda()
    out = gn_kernels.scaled_mm(A, B.T.contiguous().T, sa, sb)
    a_np = A.cpu().numpy() if kind == "int8" else bits_of(A)
    b_np = B.cpu().numpy() if kind == "int8" else bits_of(B)
    want = om.tile_scaled_mm(a_np, b_np, values_of(sa), values_of(sb), kind=kind)
    np.testing.assert_allclose(values_of(out), want, rtol=1e-2 if kind == "int8" else 1.6e-2, atol=1e-4)
    assert nv.device_status() == 0


@pytest.mark.parametrize("mnk", [(2304, 4096, 128), (2304, 4096, 256), (200, 384, 384), (2500, 3968, 512)])
@pytest.mark.parametrize("kind", ["int8", "e4m3"])
def test_tile_scaled_mm_many_tiles_per_cta_short_reductions_and_ragged_edges(mnk, kind):
    """More tiles than SMs (a CTA walks several tiles, the partial buffers and their phases carry over from one
    tile to the next), reductions of one to four blocks (the request for the next block's first chunk has
    nothing to ask for at the last block), and M / N that end inside a tile."""
    M, N, K = mnk
    g = torch.Generator().manual_seed(M + N + K)
    if kind == "int8":
        A, B = rand_i8((M, K), 71), rand_i8((K, N), 72)
    else:
        A = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn).cuda()
        B = torch.randn(K, N, generator=g).to(torch.float8_e4m3fn).cuda()
    sa = (torch.rand(M, K // 128, generator=g) / 64 + 1e-3).bfloat16().cuda()
    sb = (torch.rand(K // 128, N // 128, generator=g) / 64 + 1e-3).bfloat16().cuda()
    out = gn_kernels.scaled_mm(A, B.T.contiguous().T, sa, sb)
    a_np = A.cpu().numpy() if kind == "int8" else bits_of(A)
    b_np = B.cpu().numpy() if kind == "int8" else bits_of(B)
    want = om.tile_scaled_mm(a_np, b_np, values_of(sa), values_of(sb), kind=kind)
    np.testing.assert_allclose(values_of(out), want, rtol=1e-2 if kind == "int8" else 1.6e-2, atol=1e-4)
    assert nv.device_status() == 0
    out2 = gn_kernels.scaled_mm(A, B.T.contiguous().T, sa, sb)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("mnk", [(1024, 1024, 32768), (256, 256, 8192), (2048, 256, 16384), (300, 520, 12288), (128, 256, 8192)])
@pytest.mark.parametrize("layout", ["A@B.T", "A.T@B"])
def test_split_k_is_bit_exact(mnk, layout, cta_group):
    """Small outputs with long reductions (grad-weight shapes) split K across CTAs; integer partials
    add exactly, so int32 and scaled bf16 results equal the oracle bit for bit."""
    M, N, K = mnk
    assert nv.load().qt_gemm_workspace_bytes(M, N, K) >= 0
    A, B = rand_i8((M, K), 61), rand_i8((K, N), 62)
    g = torch.Generator().manual_seed(63)
    sa = (torch.randn(M, 1, generator=g) / 128).bfloat16().cuda()
    sb = (torch.randn(1, N, generator=g) / 128).bfloat16().cuda()
    a, b = to_layout(A, B, layout)
    acc = om.int8_mm(A.cpu().numpy(), B.cpu().numpy())
    np.testing.assert_array_equal(gn_kernels.int8_mm(a, b).cpu().numpy(), acc)
    want = om.round_to_bf16(((acc.astype(np.float32) * values_of(sa)).astype(np.float32) * values_of(sb)).astype(np.float32))
    np.testing.assert_array_equal(values_of(gn_kernels.scaled_mm(a, b, sa, sb)), want)
    assert nv.device_status() == 0


def test_split_k_is_used_for_grad_weight_shapes():
    assert nv.load().qt_gemm_workspace_bytes(1024, 1024, 32768) > 0
    assert nv.load().qt_gemm_workspace_bytes(8192, 8192, 8192) == 0
    assert nv.load().qt_gemm_workspace_bytes(32768, 1024, 1024) == 0


def test_a_wait_that_nothing_satisfies_gives_up_and_reports():
    """The kernels' mbarrier waits are bounded: a warp waiting on a barrier nobody arrives on returns
    after its limit with a code in the device status word, the context stays usable, and the word is
    clean again afterwards."""
    import ctypes

    from gn_kernels import _native as nv

    seen = ctypes.c_int(0)
    nv.check(nv.load().qt_selftest_wait_timeout(ctypes.byref(seen), 0))
    assert seen.value == 0x7E57
    assert nv.device_status() == 0
    a = torch.randint(-128, 127, (256, 256), dtype=torch.int8, device="cuda")
    out = gn_kernels.int8_mm(a, a.T)
    assert torch.equal(out.cpu(), torch._int_mm(a.cpu(), a.cpu().T.contiguous()))


def test_a_recorded_wait_failure_raises_from_the_next_gemm_call():
    """A kernel that gave up on a wait copies its code into a pinned host word; the operators read that
    word after every GEMM launch (no synchronisation) and raise RuntimeError. Here the self-test leaves
    the code set, so the next scaled_mm call must raise, and the call after that must work again."""
    import ctypes

    from gn_kernels import _native as nv

    a = torch.randint(-128, 127, (256, 256), dtype=torch.int8, device="cuda")
    sa = torch.ones(256, 1, dtype=torch.bfloat16, device="cuda")
    sb = torch.ones(1, 256, dtype=torch.bfloat16, device="cuda")
    gn_kernels.scaled_mm(a, a.T, sa, sb)   # sets up the status block
    seen = ctypes.c_int(0)
    nv.check(nv.load().qt_selftest_wait_timeout(ctypes.byref(seen), 1))
    assert seen.value == 0x7E57
    peek = ctypes.c_int(0)
    nv.check(nv.load().qt_device_status_peek(ctypes.byref(peek)))
    assert peek.value == 0x7E57
    with pytest.raises(RuntimeError, match="bounded wait"):
        gn_kernels.scaled_mm(a, a.T, sa, sb)
    assert nv.device_status() == 0
    out = gn_kernels.scaled_mm(a, a.T, sa, sb)
    ref = torch._int_mm(a.cpu(), a.cpu().T.contiguous()).float().bfloat16()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("kinds", [("e5m2", "e5m2"), ("e4m3", "e5m2"), ("e5m2", "e4m3")])
@pytest.mark.parametrize("layout", ["A@B.T", "A.T@B.T"])
def test_scaled_mm_fp8_e5m2_and_mixed_formats(kinds, layout):
    """The other FP8 format scaled_mm accepts (kernels/gn_kernels/triton_mm.py:359-361), alone and mixed
    with e4m3, against the oracle's decode + fp32 product; also the layout with both operands MN-major."""
    M, N, K = 256, 384, 512
    g = torch.Generator().manual_seed(77)
    td = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
    A8 = torch.randn(M, K, generator=g).to(td[kinds[0]]).cuda()
    B8 = torch.randn(K, N, generator=g).to(td[kinds[1]]).cuda()
    sa = (torch.rand(M, 1, generator=g) / 64 + 1e-3).bfloat16().cuda()
    sb = (torch.rand(1, N, generator=g) / 64 + 1e-3).bfloat16().cuda()
    a, b = to_layout(A8, B8, layout)
    out = gn_kernels.scaled_mm(a, b, sa, sb)
    want = om.scaled_mm(bits_of(A8), bits_of(B8), values_of(sa), values_of(sb), kind="/".join(kinds))
    np.testing.assert_allclose(values_of(out), want, rtol=1e-2, atol=1e-4)


def test_scaled_mm_fp8_both_operands_mn_major():
    M, N, K = 384, 256, 640
    g = torch.Generator().manual_seed(78)
    A8 = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn).cuda()
    B8 = torch.randn(K, N, generator=g).to(torch.float8_e4m3fn).cuda()
    sa = (torch.rand(M, 1, generator=g) / 64 + 1e-3).bfloat16().cuda()
    sb = (torch.rand(1, N, generator=g) / 64 + 1e-3).bfloat16().cuda()
    a, b = to_layout(A8, B8, "A.T@B.T")
    want = om.scaled_mm(bits_of(A8), bits_of(B8), values_of(sa), values_of(sb), kind="e4m3")
    np.testing.assert_allclose(values_of(gn_kernels.scaled_mm(a, b, sa, sb)), want, rtol=1e-2, atol=1e-4)


@pytest.mark.parametrize("size", [2048, 4096])
@pytest.mark.parametrize("layout", ["A@B.T", "A@B", "A.T@B"])
def test_sweep_sizes_int32_exact_on_sampled_rows(size, layout):
    """The middle sizes of the reference's benchmark grid (benchmark_mm.py:70-76): exact int32 accumulators
    on sampled rows against the oracle, the scaled output equal to the accumulator times power-of-two
    scales, and the same bits on a second run."""
    A, B = rand_i8((size, size), 5 + size), rand_i8((size, size), 6 + size)
    a, b = to_layout(A, B, layout)
    acc = gn_kernels.int8_mm(a, b)
    rows = torch.tensor([0, 127, 128, size // 2 + 3, size - 1], device="cuda")
    np.testing.assert_array_equal(acc[rows].cpu().numpy(), om.int8_mm(A[rows].cpu().numpy(), B.cpu().numpy()))
    sa = torch.full((size, 1), 2.0 ** -6, dtype=torch.bfloat16, device="cuda")
    sb = torch.full((1, size), 2.0 ** -8, dtype=torch.bfloat16, device="cuda")
    out = gn_kernels.scaled_mm(a, b, sa, sb)
    assert torch.equal(out, (acc.float() * 2.0 ** -14).bfloat16())
    assert torch.equal(gn_kernels.scaled_mm(a, b, sa, sb), out)
    assert torch.equal(gn_kernels.int8_mm(a, b), acc)


def test_transposed_output_form_is_bit_identical():
    """scaled_mm_t writes (A @ B)^T directly with the column scale applied first: same bits as transposing
    the ordinary result (grad-weight lands in the weight's layout without a strided copy), split-K shapes included."""
    for (M, N, K) in [(256, 384, 512), (1024, 512, 8192), (2048, 256, 32768)]:
        A, B = rand_i8((M, K), 91 + M), rand_i8((N, K), 92 + N)
        g = torch.Generator().manual_seed(M + N)
        sa = (torch.rand(M, 1, generator=g) / 64 + 1e-3).bfloat16().cuda()
        sb = (torch.rand(1, N, generator=g) / 64 + 1e-3).bfloat16().cuda()
        ref = gn_kernels.scaled_mm(A, B.T, sa, sb)
        out_t = gn_kernels.scaled_mm_t(A, B.T, sa, sb)
        assert out_t.shape == (N, M) and out_t.is_contiguous()
        assert torch.equal(out_t, ref.T)


def test_outputs_stay_inside_their_buffers():
    """Guard bands around every output of a GEMM and of the quantize kernels stay untouched (the check a
    memory checker would make), on shapes that exercise ragged edges."""
    def guarded(shape, dtype, fill):
        n = int(np.prod(shape))
        pad = 4096 // torch.empty((), dtype=dtype).element_size()
        buf = torch.full((n + 2 * pad,), fill, dtype=dtype, device="cuda")
        return buf, buf[pad:pad + n].view(shape), pad

    import ctypes

    M, N, K = 300, 520, 272
    A, B = rand_i8((M, K + 16 - K % 16), 3)[:, :K], rand_i8((N, K + 16 - K % 16), 4)[:, :K]
    cbuf, C, pad = guarded((M, N), torch.int32, 0x5A5A5A5A)
    nv.check(nv.load().qt_int8_mm(A.data_ptr(), A.stride(0), 1, B.data_ptr(), 1, B.stride(0), C.data_ptr(), N, M, N, K,
                                  nv.stream_ptr(A.device)))
    torch.cuda.synchronize()
    assert (cbuf[:pad] == 0x5A5A5A5A).all() and (cbuf[-pad:] == 0x5A5A5A5A).all()
    np.testing.assert_array_equal(C.cpu().numpy(), om.int8_mm(A.cpu().numpy(), B.cpu().numpy().T))

    x = randn_bf16((333, 776), seed=8)
    qbuf, q, qpad = guarded((333, 776), torch.int8, 0x5A)
    sbuf, s, spad = guarded((333, 1), torch.bfloat16, 7.0)
    nv.check(nv.load().qt_quantize_rowwise(x.data_ptr(), nv.QT_BF16, 333, 776, 776, q.data_ptr(), nv.QT_I8, s.data_ptr(), nv.QT_BF16,
                                           1e-12, 0, 0, 0, nv.stream_ptr(x.device)))
    tbuf, qt, tpad = guarded((776, 333), torch.int8, 0x5A)
    cs_buf, cs, cpad = guarded((776, 1), torch.bfloat16, 7.0)
    colmax = gn_kernels.col_absmax(x)
    nv.check(nv.load().qt_quantize_colwise_t(x.data_ptr(), nv.QT_BF16, 333, 776, 776, colmax.data_ptr(), qt.data_ptr(), nv.QT_I8,
                                             cs.data_ptr(), nv.QT_BF16, 1e-12, 0, 0, 0, nv.stream_ptr(x.device)))
    torch.cuda.synchronize()
    for buf, p_, fill in ((qbuf, qpad, 0x5A), (tbuf, tpad, 0x5A)):
        assert (buf[:p_] == fill).all() and (buf[-p_:] == fill).all()
    for buf, p_ in ((sbuf, spad), (cs_buf, cpad)):
        assert (buf[:p_] == 7.0).all() and (buf[-p_:] == 7.0).all()
    oq, os_ = om.quantize_rowwise(values_of(x))
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    oqt, _ = om.quantize_colwise_t(values_of(x))
    np.testing.assert_array_equal(qt.cpu().numpy(), oqt)


@pytest.mark.parametrize("mnk", [(256, 512, 256), (1024, 1536, 1024), (300, 200, 264), (16448, 1536, 1536), (128, 256, 4096)])
def test_bf16_mm_with_column_scale_epilogue(mnk, cta_group):
    """The INT8 weight-only forward (reference: subclasses/int8.py:147): a bf16 matmul on the widened int8 weight,
    then a bf16 multiply by the per-channel scale, as one tcgen05 GEMM. Against the two-step form evaluated in
    fp32 with both roundings: identical up to the fp32 summation order (1e-2 relative, most elements equal)."""
    M, N, K = mnk
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w_i8 = torch.randint(-127, 128, (N, K), dtype=torch.int8, generator=g).cuda()
    scale = (torch.rand(N, generator=g) / 64 + 1e-3).bfloat16().cuda()
    w = w_i8.to(torch.bfloat16)
    assert gn_kernels.bf16_mm_colscale_supported(x, w, scale)
    out = gn_kernels.bf16_mm_colscale(x, w, scale)
    ref = ((x.float() @ w.float().T).bfloat16().float() * scale.float()).bfloat16()
    eager = (x @ w.T) * scale
    # A different fp32 summation order can move the first rounding by one bf16 step, which the second rounding
    # can turn into two (2^-6 relative at most); that happens to a handful of elements per million. The
    # north-star tolerance of 1e-2 relative holds for all but those, and the mean error is far below it.
    floor = 1e-4 * ref.float().abs().max().item()
    for other in (ref, eager):
        torch.testing.assert_close(out.float(), other.float(), rtol=2.0 ** -6, atol=floor)
        rel = (out.float() - other.float()).abs() / (other.float().abs() + floor)
        assert (rel > 1e-2).float().mean().item() < 1e-5
    assert (out == ref).float().mean().item() > 0.97
    assert nv.device_status() == 0


@pytest.mark.parametrize("group_m", [1, 3, 32])
def test_rasterisation_group_height_does_not_change_results(group_m):
    """The order in which the persistent grid visits output tiles is a tuning choice (how tall a group of
    row-tiles sweeps the columns): exact int32 results for any height, ragged tile counts included."""
    A, B = rand_i8((1300, 640), 7), rand_i8((640, 1100), 8)
    want = om.int8_mm(A.cpu().numpy(), B.cpu().numpy())
    nv.check(nv.load().qt_set_gemm_group_m(group_m))
    try:
        np.testing.assert_array_equal(gn_kernels.int8_mm(A, B).cpu().numpy(), want)
    finally:
        nv.check(nv.load().qt_set_gemm_group_m(0))
    assert nv.device_status() == 0
