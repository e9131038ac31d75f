"""GPU parity of the tcgen05 GEMM (bf16 and e4m3 operands, fp32 accumulation in tensor memory) through
the C ABI, against the oracle's float64 product of the same rounded operands."""
import numpy as np
import pytest

from oracle import bf_oracle as O
from tests.test_gpu_a_ops import gemm

pytestmark = pytest.mark.gpu


def operands(rng, m, n, k, scale=1.0):
    a = O.round_bf16(rng.standard_normal((m, k)).astype(np.float32) * scale)
    b = O.round_bf16(rng.standard_normal((k, n)).astype(np.float32) * scale)
    return a, b


def rel_err(got, want):
    return float(np.max(np.abs(got - want)) / (np.max(np.abs(want)) + 1e-30))


# fp32 accumulation of exactly representable products: only the summation order differs from float64
ACC_TOL = 2e-5


@pytest.mark.parametrize("m,n,k", [
    (128, 256, 64),      # one tile, one k-slice
    (128, 256, 512),     # several trips round the 4-stage ring
    (256, 512, 128),     # 2 x 2 tiles
    (100, 40, 72),       # ragged M, N, K (zero-filled by TMA, masked in the epilogue)
    (1, 8, 8),           # smallest shape the tensor-core kernel takes
    (300, 264, 136),     # N tail of 8 columns
])
def test_bf16_nk_matches_oracle(gpu, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a, b = operands(rng, m, n, k)
    want = O.matmul(a, b, exact_order=False)
    got = gemm(gpu, a, np.ascontiguousarray(b.T), gpu.BF16, gpu.B_NK)
    assert rel_err(got, want) <= ACC_TOL


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (200, 328, 200), (64, 64, 256)])
def test_bf16_kn_layout_matches_oracle(gpu, m, n, k):
    # B in the reference's own [K, N] layout: consumed as an MN-major tensor-core operand
    rng = np.random.default_rng(m + n + k + 1)
    a, b = operands(rng, m, n, k)
    want = O.matmul(a, b, exact_order=False)
    got = gemm(gpu, a, b, gpu.BF16, gpu.B_KN)
    assert rel_err(got, want) <= ACC_TOL


def test_small_integer_products_are_exact(gpu):
    # the reference's bf16 GEMM test uses small integers, whose products and sums are exact
    rng = np.random.default_rng(3)
    a = rng.integers(-4, 5, size=(128, 128)).astype(np.float32)
    b = rng.integers(-4, 5, size=(128, 64)).astype(np.float32)
    got = gemm(gpu, a, np.ascontiguousarray(b.T), gpu.BF16, gpu.B_NK)
    assert np.array_equal(got, a @ b)
    assert np.array_equal(gemm(gpu, a, b, gpu.BF16, gpu.B_KN), a @ b)


def test_persistent_schedule_many_tiles(gpu):
    # more tiles than SMs: every CTA walks several tiles through both accumulator buffers
    rng = np.random.default_rng(4)
    m, n, k = 128 * 20, 256 * 9, 192
    a, b = operands(rng, m, n, k)
    want = O.matmul(a, b, exact_order=False)
    got = gemm(gpu, a, np.ascontiguousarray(b.T), gpu.BF16, gpu.B_NK)
    assert rel_err(got, want) <= ACC_TOL
    # N-tile grouping with a remainder group (more than 16 N-tiles)
    m, n, k = 256, 256 * 21, 64
    a, b = operands(rng, m, n, k)
    got = gemm(gpu, a, np.ascontiguousarray(b.T), gpu.BF16, gpu.B_NK)
    assert rel_err(got, O.matmul(a, b, exact_order=False)) <= ACC_TOL


@pytest.mark.parametrize("c_dtype_name", ["f32", "bf16"])
def test_epilogues(gpu, c_dtype_name):
    c_dtype = gpu.F32 if c_dtype_name == "f32" else gpu.BF16
    rng = np.random.default_rng(5)
    m, n, k = 200, 264, 136
    a, b = operands(rng, m, n, k, scale=0.3)
    bt = np.ascontiguousarray(b.T)
    bias = rng.standard_normal(n).astype(np.float32)
    res = O.round_bf16(rng.standard_normal((m, n)).astype(np.float32))
    base = O.matmul(a, b, exact_order=False)
    out_round = (lambda x: x) if c_dtype == gpu.F32 else O.round_bf16
    tol = 1e-5 if c_dtype == gpu.F32 else 2.0 ** -8

    def close(got, want):
        return np.max(np.abs(got - out_round(want)) / (np.abs(want) + 1.0)) <= tol

    assert close(gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype), base)
    assert close(gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype, "bias", bias=bias), base + bias)
    assert close(gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype, "bias_silu", bias=bias), O.silu(base + bias))
    assert close(gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype, "bias_residual", bias=bias, residual=res),
                 base + bias + res)
    assert close(gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype, "residual", residual=res, alpha=0.25),
                 base * 0.25 + res)
    if c_dtype == gpu.F32:
        got = gemm(gpu, a, bt, gpu.BF16, gpu.B_NK, c_dtype, "bias", bias=bias, round_c=1)
        # on the bf16 grid, and within one bf16 step of the rounded float64 result (near-ties may round apart)
        assert np.array_equal(got, O.round_bf16(got))
        assert np.max(np.abs(got - (base + bias)) / (np.abs(base + bias) + 1.0)) <= 2.0 ** -8


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (100, 72, 208), (256, 512, 384)])
def test_fp8_matches_oracle(gpu, m, n, k):
    rng = np.random.default_rng(m + k)
    a = O.e4m3_round_hw(rng.standard_normal((m, k)).astype(np.float32) * 4)
    b = O.e4m3_round_hw(rng.standard_normal((k, n)).astype(np.float32) * 4)
    want = O.matmul(a, b, exact_order=False)
    got = gemm(gpu, a, np.ascontiguousarray(b.T), gpu.FP8_E4M3, gpu.B_NK, alpha=0.5)
    assert rel_err(got, want * 0.5) <= ACC_TOL


@pytest.mark.parametrize("dtype_name", ["bf16", "fp8"])
def test_wide_tile_path_with_ragged_edges(gpu, dtype_name):
    # enough 256 x 512 tiles (>= one per CTA pair) and K >= 1024 select the 512-column accumulator; M and N are
    # ragged so the last tile row / column is partly outside, and every CTA pair walks more than one tile
    rng = np.random.default_rng(11)
    m, n, k = 256 * 12 - 60, 512 * 8 - 248, 1024
    if dtype_name == "bf16":
        a, b = operands(rng, m, n, k, scale=0.5)
        ab = gpu.BF16
    else:
        a = O.e4m3_round_hw(rng.standard_normal((m, k)).astype(np.float32) * 2)
        b = O.e4m3_round_hw(rng.standard_normal((k, n)).astype(np.float32) * 2)
        ab = gpu.FP8_E4M3
    bias = rng.standard_normal(n).astype(np.float32)
    res = O.round_bf16(rng.standard_normal((m, n)).astype(np.float32))
    want = O.matmul(a, b, exact_order=False) + bias + res
    got = gemm(gpu, a, np.ascontiguousarray(b.T), ab, gpu.B_NK, gpu.F32, "bias_residual", bias=bias, residual=res)
    assert rel_err(got, want) <= ACC_TOL


def test_fp8_scaled_gemm_definition(gpu):
    # the project's `compute fp8.e4m3` arithmetic end to end: amax -> scale -> e4m3 -> GEMM -> rescale
    rng = np.random.default_rng(6)
    m, n, k = 96, 80, 160
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    want = O.fp8_scaled_matmul(a, w)
    sa = np.float32(448.0) / np.abs(a).max()
    sw = np.float32(448.0) / np.abs(w).max()
    got = gemm(gpu, a * sa, np.ascontiguousarray((w * sw).T), gpu.FP8_E4M3, gpu.B_NK,
               alpha=float(np.float32(1.0) / (sa * sw)))
    assert rel_err(got, want) <= 1e-5
    # and it is a sane approximation of the fp32 product
    assert rel_err(got, O.matmul(a, w, exact_order=False)) <= 0.08


def test_linearity_at_benchmark_width(gpu):
    # size-independent property at the 2B-class layer width: (A1 + A2) W = A1 W + A2 W on dyadic data
    rng = np.random.default_rng(7)
    m, n, k = 512, 2048, 2048
    a1 = rng.integers(-2, 3, size=(m, k)).astype(np.float32)
    a2 = rng.integers(-2, 3, size=(m, k)).astype(np.float32)
    w = (rng.integers(-2, 3, size=(k, n)) / 4).astype(np.float32)
    wt = np.ascontiguousarray(w.T)
    lhs = gemm(gpu, a1 + a2, wt, gpu.BF16, gpu.B_NK)
    rhs = gemm(gpu, a1, wt, gpu.BF16, gpu.B_NK) + gemm(gpu, a2, wt, gpu.BF16, gpu.B_NK)
    assert np.array_equal(lhs, rhs)
    assert np.array_equal(lhs[:4], ((a1 + a2)[:4].astype(np.float64) @ w.astype(np.float64)).astype(np.float32))
