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


@pytest.mark.parametrize("m,n,k,epilogue,wide", [
    (300, 264, 136, "none", False),        # ragged rows and an 8-column N tail
    (512, 512, 256, "bias_silu", False),
    (384, 1024, 1024, "bias_residual", True),   # the 512-column tile (tests lower its switch-over depth to K = 1024)
])
def test_rmsnorm_folded_into_the_gemm(gpu, m, n, k, epilogue, wide):
    """C = epilogue(rmsnorm(A) W^T) computed as row-scaled (A W^T): the GEMM reads the un-normalised A and divides
    row i by sqrt(mean(A_i^2) + eps) in its epilogue. Checked against float64 arithmetic on the same bf16
    operands; the sums of squares of the stored rows come back for the next norm."""
    rng = np.random.default_rng(m + n + k)
    a = O.round_bf16((rng.standard_normal((m, k)) * rng.uniform(0.2, 5.0, size=(m, 1))).astype(np.float32))
    w = O.round_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.1)
    bias = rng.standard_normal(n).astype(np.float32)
    res = O.round_bf16(rng.standard_normal((m, n)).astype(np.float32))
    d_a, d_w = gpu.upload(a, gpu.BF16), gpu.upload(w, gpu.BF16)
    d_bias, d_res = gpu.DeviceBuffer.from_numpy(bias), gpu.upload(res, gpu.BF16)
    d_ss = gpu.DeviceBuffer(m * 4)
    gpu.check(gpu.lib().bfb_row_sum_squares(d_a.ptr, gpu.BF16, d_ss.ptr, m, k, None))
    ss = d_ss.to_numpy(np.float32, (m,))
    want_ss = np.sum(a.astype(np.float64) ** 2, axis=1)
    assert np.max(np.abs(ss - want_ss) / want_ss) <= 1e-5
    d_c = gpu.DeviceBuffer(m * n * 2)
    parts = (n + 127) // 128
    d_out_ss = gpu.DeviceBuffer(parts * m * 4)
    d_out_mx = gpu.DeviceBuffer(parts * m * 4)
    status = gpu.DeviceBuffer.zeros(4)
    epi = gpu.EPI[epilogue]
    gpu.check(gpu.lib().bfb_gemm_rmsnorm(d_a.ptr, d_w.ptr, d_c.ptr, m, n, k, gpu.BF16, gpu.BF16, epi,
                                         d_bias.ptr if epilogue != "none" else None,
                                         d_res.ptr if epilogue == "bias_residual" else None,
                                         d_ss.ptr, 1, 1e-6, d_out_ss.ptr, d_out_mx.ptr, status.ptr, None))
    got = gpu.download(d_c, gpu.BF16, (m, n))
    assert status.to_numpy(np.int32, (1,))[0] == 0
    normed = a.astype(np.float64) / np.sqrt(want_ss / k + 1e-6)[:, None]
    want = normed @ w.astype(np.float64).T
    if epilogue != "none":
        want = want + bias
    if epilogue == "bias_silu":
        want = want / (1.0 + np.exp(-want))
    if epilogue == "bias_residual":
        want = want + res
    # one rounding to bf16 on top of fp32 accumulation
    assert np.max(np.abs(got - want) / (np.abs(want) + 0.05)) <= 2.0 ** -8 + 1e-3
    out_ss = d_out_ss.to_numpy(np.float32, (parts, m))
    padded = np.zeros((m, parts * 128))
    padded[:, :n] = got.astype(np.float64) ** 2
    stored = padded.reshape(m, parts, 128).sum(axis=2).T          # [parts][m], one figure per 128 columns
    assert np.max(np.abs(out_ss - stored) / (stored + 1e-30)) <= 1e-5
    out_mx = d_out_mx.to_numpy(np.float32, (parts, m))
    padded_abs = np.zeros((m, parts * 128), np.float32)
    padded_abs[:, :n] = np.abs(got)
    assert np.array_equal(out_mx, padded_abs.reshape(m, parts, 128).max(axis=2).T)     # exact: maxima of stored values
    # those parts drive the next GEMM exactly like the one-part sums of a separate pass over C
    d_c2, d_c3 = gpu.DeviceBuffer(m * 64 * 2), gpu.DeviceBuffer(m * 64 * 2)
    w2 = O.round_bf16(rng.standard_normal((64, n)).astype(np.float32) * 0.1)
    d_w2 = gpu.upload(w2, gpu.BF16)
    gpu.check(gpu.lib().bfb_gemm_rmsnorm(d_c.ptr, d_w2.ptr, d_c2.ptr, m, 64, n, gpu.BF16, gpu.BF16, gpu.EPI["none"], None,
                                         None, d_out_ss.ptr, parts, 1e-6, None, None, status.ptr, None))
    d_one = gpu.DeviceBuffer(m * 4)
    gpu.check(gpu.lib().bfb_row_sum_squares(d_c.ptr, gpu.BF16, d_one.ptr, m, n, None))
    gpu.check(gpu.lib().bfb_gemm_rmsnorm(d_c.ptr, d_w2.ptr, d_c3.ptr, m, 64, n, gpu.BF16, gpu.BF16, gpu.EPI["none"], None,
                                         None, d_one.ptr, 1, 1e-6, None, None, status.ptr, None))
    got2, got3 = gpu.download(d_c2, gpu.BF16, (m, 64)), gpu.download(d_c3, gpu.BF16, (m, 64))
    assert np.max(np.abs(got2 - got3) / (np.abs(got3) + 0.05)) <= 2.0 ** -7
    # and the e4m3 quantisation of rmsnorm(C): from the epilogue's statistics (C read once) as from two passes over C
    winv = gpu.DeviceBuffer.from_numpy(np.array([0.5], np.float32))
    q_plain, s_plain = gpu.DeviceBuffer(m * n), gpu.DeviceBuffer.zeros(12)
    q_stats, s_stats = gpu.DeviceBuffer(m * n), gpu.DeviceBuffer.zeros(12)
    gpu.check(gpu.lib().bfb_rmsnorm_quantize_e4m3(d_c.ptr, m, n, 1e-6, q_plain.ptr, s_plain.ptr, winv.ptr, None))
    gpu.check(gpu.lib().bfb_rmsnorm_quantize_e4m3_from_stats(d_c.ptr, m, n, 1e-6, q_stats.ptr, s_stats.ptr, winv.ptr,
                                                             d_out_ss.ptr, d_out_mx.ptr, parts, None))
    sp, st = s_plain.to_numpy(np.float32, (3,)), s_stats.to_numpy(np.float32, (3,))
    assert np.max(np.abs(sp - st) / sp) <= 2.0 ** -7            # the maximum may sit one bf16 step apart
    qa, qb = gpu.download(q_plain, gpu.FP8_E4M3, (m, n)), gpu.download(q_stats, gpu.FP8_E4M3, (m, n))
    if np.array_equal(sp, st):
        # a last-bit difference in a row's 1 / rms may move single values across a rounding boundary
        assert np.mean(qa != qb) <= 2e-3 and np.max(np.abs(qa - qb) / (np.abs(qa) + 2.0 ** -6)) <= 0.13


def test_row_statistics_need_the_tensor_core_kernel(gpu):
    # rows of 60 bf16 values are not 16-byte multiples: the CUDA-core kernel would run, and it has no row statistics
    a = np.ones((64, 60), np.float32)
    d_a, d_w, d_c = gpu.upload(a, gpu.BF16), gpu.upload(a, gpu.BF16), gpu.DeviceBuffer(64 * 64 * 2)
    d_ss = gpu.DeviceBuffer.zeros(64 * 4)
    rc = gpu.lib().bfb_gemm_rmsnorm(d_a.ptr, d_w.ptr, d_c.ptr, 64, 64, 60, gpu.BF16, gpu.BF16, gpu.EPI["none"], None, None,
                                    d_ss.ptr, 1, 1e-6, None, None, None, None)
    assert rc == gpu.UNSUPPORTED


def test_folded_rmsnorm_gives_the_same_bits_for_any_number_of_rows(gpu):
    """A sequence must come out the same alone (few rows) and inside a batch (many rows, other tile shapes)."""
    rng = np.random.default_rng(77)
    m, n, k = 640, 512, 1024
    a = O.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = O.round_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.1)
    d_w = gpu.upload(w, gpu.BF16)

    def run(rows):
        d_a = gpu.upload(a[:rows], gpu.BF16)
        d_ss, d_c = gpu.DeviceBuffer(rows * 4), gpu.DeviceBuffer(rows * n * 2)
        d_out = gpu.DeviceBuffer(4 * rows * 4)
        gpu.check(gpu.lib().bfb_row_sum_squares(d_a.ptr, gpu.BF16, d_ss.ptr, rows, k, None))
        gpu.check(gpu.lib().bfb_gemm_rmsnorm(d_a.ptr, d_w.ptr, d_c.ptr, rows, n, k, gpu.BF16, gpu.BF16, gpu.EPI["none"],
                                             None, None, d_ss.ptr, 1, 1e-6, d_out.ptr, None, None, None))
        return gpu.download(d_c, gpu.BF16, (rows, n)), d_out.to_numpy(np.float32, (4, rows))

    whole, whole_ss = run(m)
    for rows in (1, 100, 128, 300):
        part, part_ss = run(rows)
        assert np.array_equal(part, whole[:rows]) and np.array_equal(part_ss, whole_ss[:, :rows])


@pytest.mark.parametrize("m,n,k", [(4133, 3080, 512), (9000, 1024, 256), (300, 512, 128)])
def test_tiles_drawn_from_a_counter_give_the_same_bits(gpu, m, n, k):
    """The CTA-pair GEMM with its tiles handed out by atomicAdd (the mode for GEMMs that share the SMs with another
    stream's kernel), also on a grid sized for fewer SMs: same tiles, so every value and statistic is identical."""
    rng = np.random.default_rng(m + n + k)
    a = O.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = O.round_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.1)
    d_a, d_w = gpu.upload(a, gpu.BF16), gpu.upload(w, gpu.BF16)
    parts = (n + 127) // 128

    def run():
        d_ss, d_c = gpu.DeviceBuffer(m * 4), gpu.DeviceBuffer(m * n * 2)
        d_out = gpu.DeviceBuffer(parts * m * 4)
        gpu.check(gpu.lib().bfb_row_sum_squares(d_a.ptr, gpu.BF16, d_ss.ptr, m, k, None))
        gpu.check(gpu.lib().bfb_gemm_rmsnorm(d_a.ptr, d_w.ptr, d_c.ptr, m, n, k, gpu.BF16, gpu.BF16, gpu.EPI["none"],
                                             None, None, d_ss.ptr, 1, 1e-6, d_out.ptr, None, None, None))
        return gpu.download(d_c, gpu.BF16, (m, n)), d_out.to_numpy(np.float32, (parts, m))

    want, want_ss = run()
    try:
        for reserved in (0, 40, 146):
            gpu.set_shared_sm_mode(True, reserved)
            for _ in range(2):
                got, got_ss = run()
                assert np.array_equal(got, want) and np.array_equal(got_ss, want_ss), reserved
    finally:
        gpu.set_shared_sm_mode(False, 0)
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    ref /= np.sqrt(np.mean(a.astype(np.float64) ** 2, axis=1, keepdims=True) + 1e-6)
    assert np.max(np.abs(want - ref)) <= 2e-2 * np.max(np.abs(ref))


@pytest.mark.parametrize("m,n,k,epilogue,c_dtype", [
    (1, 264, 136, "none", "bf16"),              # one row, N tail of 8 columns, K tail
    (7, 2048, 2048, "residual", "bf16"),        # 16 column tiles x 8 K-splits
    (32, 2048, 5632, "bias_residual", "bf16"),
    (100, 512, 320, "bias_silu", "bf16"),
    (128, 1000, 512, "bias", "f32"),
    (33, 6144, 2048, "none", "bf16"),
])
def test_few_rows_gemm_matches_oracle(gpu, m, n, k, epilogue, c_dtype):
    """The generation-step GEMM (weights on the MMA's M side, K split across CTAs, partial products added in a
    fixed order) against float64 arithmetic on the same bf16 operands, with the folded rmsnorm and its statistics."""
    rng = np.random.default_rng(m * 3 + n + k)
    a = O.round_bf16((rng.standard_normal((m, k)) * rng.uniform(0.3, 3.0, size=(m, 1))).astype(np.float32))
    w = O.round_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.1)
    bias = rng.standard_normal(n).astype(np.float32)
    cd = gpu.BF16 if c_dtype == "bf16" else gpu.F32
    res = rng.standard_normal((m, n)).astype(np.float32)
    if cd == gpu.BF16:
        res = O.round_bf16(res)
    d_a, d_w = gpu.upload(a, gpu.BF16), gpu.upload(w, gpu.BF16)
    d_bias, d_res = gpu.DeviceBuffer.from_numpy(bias), gpu.upload(res, cd)
    d_ss = gpu.DeviceBuffer(m * 4)
    gpu.check(gpu.lib().bfb_row_sum_squares(d_a.ptr, gpu.BF16, d_ss.ptr, m, k, None))
    parts = (n + 127) // 128
    d_c = gpu.DeviceBuffer(m * n * (2 if cd == gpu.BF16 else 4))
    d_out_ss = gpu.DeviceBuffer(parts * m * 4)
    status = gpu.DeviceBuffer.zeros(4)
    has_bias, has_res = epilogue.startswith("bias"), epilogue.endswith("residual")
    for run in range(2):
        gpu.check(gpu.lib().bfb_gemm_few_rows(d_a.ptr, d_w.ptr, d_c.ptr, m, n, k, gpu.BF16, cd, gpu.EPI[epilogue],
                                              d_bias.ptr if has_bias else None, d_res.ptr if has_res else None, 1.0,
                                              d_ss.ptr, 1, 1e-6, d_out_ss.ptr, status.ptr, None))
        got = gpu.download(d_c, cd, (m, n))
        if run == 0:
            first = got.copy()
    assert np.array_equal(first, got)                      # no atomics: the same bits every time
    assert status.to_numpy(np.int32, (1,))[0] == 0
    ssq = np.sum(a.astype(np.float64) ** 2, axis=1)
    want = (a.astype(np.float64) / np.sqrt(ssq / k + 1e-6)[:, None]) @ w.astype(np.float64).T
    if has_bias:
        want = want + bias
    if epilogue == "bias_silu":
        want = want / (1.0 + np.exp(-want))
    if has_res:
        want = want + res
    tol = 2.0 ** -8 + 1e-3 if cd == gpu.BF16 else 1e-4
    assert np.max(np.abs(got - want) / (np.abs(want) + 0.05)) <= tol
    out_ss = d_out_ss.to_numpy(np.float32, (parts, m))
    padded = np.zeros((m, parts * 128))
    padded[:, :n] = got.astype(np.float64) ** 2
    stored = padded.reshape(m, parts, 128).sum(axis=2).T
    assert np.max(np.abs(out_ss - stored) / (stored + 1e-30)) <= 1e-5
    # a row gives the same bits whatever rows sit beside it
    if m > 1:
        d_c1 = gpu.DeviceBuffer(n * (2 if cd == gpu.BF16 else 4))
        gpu.check(gpu.lib().bfb_gemm_few_rows(d_a.ptr, d_w.ptr, d_c1.ptr, 1, n, k, gpu.BF16, cd, gpu.EPI[epilogue],
                                              d_bias.ptr if has_bias else None, d_res.ptr if has_res else None, 1.0,
                                              d_ss.ptr, 1, 1e-6, None, status.ptr, None))
        assert np.array_equal(gpu.download(d_c1, cd, (1, n)), got[:1])


def test_few_rows_gemm_e4m3_and_limits(gpu):
    rng = np.random.default_rng(5)
    m, n, k = 24, 384, 512
    a = O.e4m3_round_hw(rng.standard_normal((m, k)).astype(np.float32))
    w = O.e4m3_round_hw(rng.standard_normal((n, k)).astype(np.float32))
    d_a, d_w = gpu.upload(a, gpu.FP8_E4M3), gpu.upload(w, gpu.FP8_E4M3)
    d_c = gpu.DeviceBuffer(m * n * 4)
    gpu.check(gpu.lib().bfb_gemm_few_rows(d_a.ptr, d_w.ptr, d_c.ptr, m, n, k, gpu.FP8_E4M3, gpu.F32, gpu.EPI["none"], None,
                                          None, 0.5, None, 1, 0.0, None, None, None))
    want = 0.5 * (a.astype(np.float64) @ w.astype(np.float64).T)
    assert rel_err(gpu.download(d_c, gpu.F32, (m, n)), want) <= ACC_TOL
    rc = gpu.lib().bfb_gemm_few_rows(d_a.ptr, d_w.ptr, d_c.ptr, 129, n, k, gpu.FP8_E4M3, gpu.F32, gpu.EPI["none"], None, None,
                                     1.0, None, 1, 0.0, None, None, None)
    assert rc == gpu.INVALID_ARGUMENT
