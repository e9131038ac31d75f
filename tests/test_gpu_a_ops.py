"""GPU parity of the memory-bound kernels and the CUDA-core GEMM / attention, through the C ABI,
against the numpy oracle and the golden fixtures (outputs of the reference's CPU backend)."""
import ctypes as C

import numpy as np
import pytest

from oracle import bf_oracle as O

pytestmark = pytest.mark.gpu


def run_elementwise(bfb, op, a, b=None, c=None, cols=0):
    da = bfb.DeviceBuffer.from_numpy(a.astype(np.float32))
    db = bfb.DeviceBuffer.from_numpy(b.astype(np.float32)) if b is not None else None
    dc = bfb.DeviceBuffer.from_numpy(c.astype(np.float32)) if c is not None else None
    out = bfb.DeviceBuffer(a.size * 4)
    bfb.check(bfb.lib().bfb_elementwise(bfb.EW[op], da.ptr, db.ptr if db else None, dc.ptr if dc else None, out.ptr,
                                        a.size, cols, None))
    return out.to_numpy(np.float32, a.shape)


def test_elementwise_against_golden(gpu, golden_ops):
    g = golden_ops
    x = g["unary_x"]
    assert np.array_equal(run_elementwise(gpu, "relu", x), g["unary_relu"])
    assert np.max(np.abs(run_elementwise(gpu, "silu", x) - g["unary_silu"])) <= 1e-5   # reference test bar
    assert np.max(np.abs(run_elementwise(gpu, "gelu", x) - g["unary_gelu"])) <= 1e-5
    ab = g["mm_ab"]
    assert np.array_equal(run_elementwise(gpu, "add_bias", ab, g["lin_bias"], cols=9), g["addbias_out"])
    assert np.array_equal(run_elementwise(gpu, "add", ab, ab), ab + ab)
    res = np.ones_like(ab)
    got = run_elementwise(gpu, "add_bias_residual", ab, g["lin_bias"], res, cols=9)
    assert np.array_equal(got, (ab + g["lin_bias"]) + res)
    got = run_elementwise(gpu, "add_bias_silu", ab, g["lin_bias"], cols=9)
    assert np.max(np.abs(got - O.silu(ab + g["lin_bias"]))) <= 1e-5


@pytest.mark.parametrize("shape", [(3, 5, 300), (7, 64), (5, 2048), (2, 8192), (3, 10), (2, 9000), (5, 4096), (3, 6144),
                                   (9, 8192)])
def test_rmsnorm_matches_oracle(gpu, shape):
    x = (np.random.default_rng(sum(shape)).standard_normal(shape) * 2).astype(np.float32)
    rows, dim = int(np.prod(shape[:-1])), shape[-1]
    dx = gpu.DeviceBuffer.from_numpy(x)
    out = gpu.DeviceBuffer(x.nbytes)
    gpu.check(gpu.lib().bfb_rmsnorm(dx.ptr, gpu.F32, out.ptr, gpu.F32, rows, dim, 1e-6, None))
    got = out.to_numpy(np.float32, shape)
    assert np.max(np.abs(got - O.rmsnorm(x))) <= 1e-4      # tests/backend/cuda/ops_tests.cu:179-208
    # bf16 in / bf16 out: the rounded input normalised, rounded once more
    xb = O.round_bf16(x)
    d16 = gpu.upload(xb, gpu.BF16)
    o16 = gpu.DeviceBuffer(x.size * 2)
    gpu.check(gpu.lib().bfb_rmsnorm(d16.ptr, gpu.BF16, o16.ptr, gpu.BF16, rows, dim, 1e-6, None))
    got16 = gpu.download(o16, gpu.BF16, shape)
    want = O.rmsnorm(xb)
    assert np.max(np.abs(got16 - want) / (np.abs(want) + 1e-3)) <= 2.0 ** -7


def test_rmsnorm_golden_and_empty(gpu, golden_ops):
    x = golden_ops["unary_x"]
    dx = gpu.DeviceBuffer.from_numpy(x)
    out = gpu.DeviceBuffer(x.nbytes)
    gpu.check(gpu.lib().bfb_rmsnorm(dx.ptr, gpu.F32, out.ptr, gpu.F32, 15, 300, 1e-6, None))
    assert np.max(np.abs(out.to_numpy(np.float32, x.shape) - golden_ops["unary_rmsnorm"])) <= 1e-4
    assert gpu.lib().bfb_rmsnorm(None, gpu.F32, None, gpu.F32, 0, 300, 1e-6, None) == gpu.OK


def test_softmax_matches_golden(gpu, golden_ops):
    x = golden_ops["unary_x"]
    dx = gpu.DeviceBuffer.from_numpy(x)
    out = gpu.DeviceBuffer(x.nbytes)
    gpu.check(gpu.lib().bfb_softmax(dx.ptr, out.ptr, 15, 300, None))
    got = out.to_numpy(np.float32, x.shape)
    assert np.max(np.abs(got - golden_ops["unary_softmax"])) <= 1e-6
    assert np.allclose(got.sum(axis=-1), 1.0, atol=1e-5)


def embed(gpu, ids, table, pos, out_dtype, pos_offset=0, count_oob=True):
    B, S = ids.shape
    V, d = table.shape
    dids, dtab = gpu.DeviceBuffer.from_numpy(ids), gpu.DeviceBuffer.from_numpy(table)
    dpos = gpu.DeviceBuffer.from_numpy(pos) if pos is not None else None
    out = gpu.DeviceBuffer(B * S * d * gpu.ELEM_BYTES[out_dtype])
    oob = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_embed_pos(dids.ptr, dtab.ptr, dpos.ptr if dpos else None, out.ptr, out_dtype, B, S, V, d,
                                      pos.shape[0] if pos is not None else 0, pos_offset,
                                      oob.ptr if count_oob else None, None))
    return gpu.download(out, out_dtype, (B, S, d)), int(oob.to_numpy(np.int32, (1,))[0])


def test_embedding_and_positions_are_bit_exact(gpu, golden_ops):
    g = golden_ops
    got, bad = embed(gpu, g["emb_ids"], g["emb_table"], None, gpu.F32)
    assert bad == 0 and np.array_equal(got, g["emb_out"])
    got, _ = embed(gpu, g["emb_ids"], g["emb_table"], g["emb_pos"], gpu.F32)
    assert np.array_equal(got, g["pos_out"])
    got, _ = embed(gpu, g["emb_ids"], g["emb_table"], g["emb_pos"], gpu.F32, pos_offset=2)
    assert np.array_equal(got, g["pos_at2_out"])
    got16, _ = embed(gpu, g["emb_ids"], g["emb_table"], g["emb_pos"], gpu.BF16)
    assert np.array_equal(got16, O.round_bf16(g["pos_out"]))
    # standalone positional add on an existing tensor
    din, dpos = gpu.DeviceBuffer.from_numpy(g["emb_out"]), gpu.DeviceBuffer.from_numpy(g["emb_pos"])
    out = gpu.DeviceBuffer(g["emb_out"].nbytes)
    gpu.check(gpu.lib().bfb_add_positional(din.ptr, dpos.ptr, out.ptr, 3, 10, 24, 12, 0, None))
    assert np.array_equal(out.to_numpy(np.float32, g["emb_out"].shape), g["pos_out"])


def test_embedding_large_vectorised_and_odd_width(gpu):
    rng = np.random.default_rng(8)
    for V, d, B, S in ((1000, 2048, 3, 17), (37, 13, 2, 5)):
        table = rng.standard_normal((V, d)).astype(np.float32)
        pos = rng.standard_normal((S + 3, d)).astype(np.float32)
        ids = rng.integers(0, V, size=(B, S)).astype(np.float32)
        got, bad = embed(gpu, ids, table, pos, gpu.F32)
        want = O.add_positional_embedding(O.embedding_lookup(ids, table), pos)
        assert bad == 0 and np.array_equal(got, want)


def test_embedding_out_of_range_ids_are_counted_and_zero_filled(gpu):
    table = np.arange(12, dtype=np.float32).reshape(4, 3) + 1
    ids = np.array([[0, 4, -1, 3.4, 2.5, np.nan]], dtype=np.float32)   # lround: 3.4 -> 3, 2.5 -> 3
    got, bad = embed(gpu, ids, table, None, gpu.F32)
    assert bad == 3
    assert np.array_equal(got[0, 0], table[0]) and np.array_equal(got[0, 3], table[3]) and np.array_equal(got[0, 4], table[3])
    assert not got[0, 1].any() and not got[0, 2].any() and not got[0, 5].any()
    # positions beyond the table are rejected before any launch
    dids = gpu.DeviceBuffer.from_numpy(ids)
    st = gpu.lib().bfb_embed_pos(dids.ptr, dids.ptr, dids.ptr, dids.ptr, gpu.F32, 1, 6, 4, 3, 5, 0, None, None)
    assert st == gpu.INVALID_ARGUMENT


def test_cast_round_trips_and_amax(gpu):
    rng = np.random.default_rng(9)
    x = (rng.standard_normal(4099) * 30).astype(np.float32)
    d16 = gpu.upload(x, gpu.BF16)
    assert np.array_equal(gpu.download(d16, gpu.BF16, x.shape), O.round_bf16(x))
    amax = gpu.DeviceBuffer.zeros(4)
    src = gpu.DeviceBuffer.from_numpy(x)
    gpu.check(gpu.lib().bfb_amax(src.ptr, gpu.F32, x.size, amax.ptr, None))
    a = amax.to_numpy(np.float32, (1,))[0]
    assert a == np.abs(x).max()
    scales = gpu.DeviceBuffer(8)
    gpu.check(gpu.lib().bfb_fp8_scale_from_amax(amax.ptr, scales.ptr, None))
    s = scales.to_numpy(np.float32, (2,))
    assert s[0] == np.float32(448.0) / a and abs(s[1] * s[0] - 1) < 1e-6
    d8 = gpu.DeviceBuffer(x.size)
    gpu.check(gpu.lib().bfb_cast(src.ptr, gpu.F32, d8.ptr, gpu.FP8_E4M3, x.size, 1.0, scales.ptr, None))
    got = gpu.download(d8, gpu.FP8_E4M3, x.shape)
    assert np.array_equal(got, O.e4m3_round_hw(x * s[0]))
    # saturation and the vectorised bf16 -> e4m3 form
    big = np.array([1000.0, -1000.0, 448.0, 0.0, 1e-9, 0.3, -0.3, 17.0] * 2, dtype=np.float32)
    d8b = gpu.DeviceBuffer(big.size)
    dbig = gpu.upload(big, gpu.BF16)
    gpu.check(gpu.lib().bfb_cast(dbig.ptr, gpu.BF16, d8b.ptr, gpu.FP8_E4M3, big.size, 1.0, None, None))
    assert np.array_equal(gpu.download(d8b, gpu.FP8_E4M3, big.shape), O.e4m3_round_hw(O.round_bf16(big)))


def test_weight_prepare_transposes_and_converts(gpu):
    rng = np.random.default_rng(10)
    for k, n in ((70, 45), (64, 256)):
        w = rng.standard_normal((k, n)).astype(np.float32)
        dw = gpu.DeviceBuffer.from_numpy(w)
        out = gpu.DeviceBuffer(k * n * 2)
        gpu.check(gpu.lib().bfb_weight_prepare(dw.ptr, out.ptr, gpu.BF16, k, n, 1.0, None, None))
        assert np.array_equal(gpu.download(out, gpu.BF16, (n, k)), O.round_bf16(w.T))
        out32 = gpu.DeviceBuffer(k * n * 4)
        gpu.check(gpu.lib().bfb_weight_prepare(dw.ptr, out32.ptr, gpu.F32, k, n, 0.5, None, None))
        assert np.array_equal(out32.to_numpy(np.float32, (n, k)), w.T * np.float32(0.5))


def gemm(gpu, a, b, ab_dtype, b_layout, c_dtype=None, epilogue="none", bias=None, residual=None, alpha=1.0,
         round_c=0):
    """a [M,K] fp32 host, b fp32 host already in the requested layout; returns fp32 host result."""
    c_dtype = gpu.F32 if c_dtype is None else c_dtype
    m, k = a.shape
    n = b.shape[1] if b_layout == gpu.B_KN else b.shape[0]
    da, db = gpu.upload(a, ab_dtype), gpu.upload(b, ab_dtype)
    dbias = gpu.DeviceBuffer.from_numpy(bias.astype(np.float32)) if bias is not None else None
    dres = gpu.upload(residual, c_dtype) if residual is not None else None
    dc = gpu.DeviceBuffer(m * n * gpu.ELEM_BYTES[c_dtype])
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_gemm(da.ptr, db.ptr, dc.ptr, m, n, k, ab_dtype, b_layout, c_dtype, gpu.EPI[epilogue],
                                 dbias.ptr if dbias else None, dres.ptr if dres else None, alpha, None, round_c,
                                 status.ptr, None))
    gpu.sync()
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0, "a bounded device wait ran out"
    return gpu.download(dc, c_dtype, (m, n))


def test_fp32_gemm_known_answers_and_golden(gpu, golden_ops):
    got = gemm(gpu, np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32), gpu.F32, gpu.B_KN)
    assert got.tolist() == [[19, 22], [43, 50]]
    g = golden_ops
    got = gemm(gpu, g["mm_a"], g["mm_b"], gpu.F32, gpu.B_KN)
    assert np.max(np.abs(got - g["mm_ab"])) <= 1e-5      # fused multiply-add vs separate rounding only
    got = gemm(gpu, g["mm_a"], g["mm_b"], gpu.F32, gpu.B_KN, epilogue="bias", bias=g["lin_bias"])
    assert np.max(np.abs(got - g["lin_out"].reshape(17, 9))) <= 1e-5
    got = gemm(gpu, g["mm_a"], np.ascontiguousarray(g["mm_b"].T), gpu.F32, gpu.B_NK)
    assert np.max(np.abs(got - g["mm_ab"])) <= 1e-5
    # matmulTransposeB
    da, dc_ = gpu.DeviceBuffer.from_numpy(g["mm_a"]), gpu.DeviceBuffer.from_numpy(g["mm_c"])
    out = gpu.DeviceBuffer(17 * 21 * 4)
    gpu.check(gpu.lib().bfb_matmul_transpose_b(da.ptr, dc_.ptr, out.ptr, 17, 21, 33, None))
    assert np.max(np.abs(out.to_numpy(np.float32, (17, 21)) - g["mm_act"])) <= 1e-5


@pytest.mark.parametrize("m,n,k", [(130, 70, 200), (64, 64, 64), (1, 5, 3), (257, 129, 31)])
def test_fp32_gemm_epilogues(gpu, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32)
    bias, res = rng.standard_normal(n).astype(np.float32), rng.standard_normal((m, n)).astype(np.float32)
    base = O.matmul(a, b, exact_order=False)
    tol = 1e-3     # non-square vs CPU bar of the reference (ops_tests.cu:53-83)
    assert np.max(np.abs(gemm(gpu, a, b, gpu.F32, gpu.B_KN) - base)) <= tol
    assert np.max(np.abs(gemm(gpu, a, b, gpu.F32, gpu.B_KN, epilogue="bias_silu", bias=bias) - O.silu(base + bias))) <= tol
    got = gemm(gpu, a, b, gpu.F32, gpu.B_KN, epilogue="bias_residual", bias=bias, residual=res)
    assert np.max(np.abs(got - (base + bias + res))) <= tol
    got = gemm(gpu, a, b, gpu.F32, gpu.B_KN, epilogue="residual", residual=res, alpha=0.5)
    assert np.max(np.abs(got - (base * 0.5 + res))) <= tol


def test_cuda_core_gemm_takes_unaligned_bf16_and_fp8(gpu):
    # K and N that the tensor-core kernel's 16-byte rules exclude still work, with the same arithmetic contract
    rng = np.random.default_rng(12)
    a, b = rng.standard_normal((33, 37)).astype(np.float32), rng.standard_normal((37, 21)).astype(np.float32)
    want = O.matmul(O.round_bf16(a), O.round_bf16(b), exact_order=False)
    assert np.max(np.abs(gemm(gpu, a, b, gpu.BF16, gpu.B_KN) - want)) <= 1e-3
    a8, b8 = O.e4m3_round_hw(a), O.e4m3_round_hw(b)
    got = gemm(gpu, a8, np.ascontiguousarray(b8.T), gpu.FP8_E4M3, gpu.B_NK)
    assert np.max(np.abs(got - O.matmul(a8, b8, exact_order=False))) <= 1e-3


def attention(gpu, q, k, v, heads, dtype, old_len=0, causal=1, scale=None):
    B, new_len, dim = q.shape
    total = k.shape[1]
    hd = dim // heads
    scale = 1.0 / np.sqrt(np.float32(hd)) if scale is None else scale
    dq, dk, dv = gpu.upload(q, dtype), gpu.upload(k, dtype), gpu.upload(v, dtype)
    out = gpu.DeviceBuffer(q.size * gpu.ELEM_BYTES[dtype])
    dm, dl = gpu.DeviceBuffer(B * heads * new_len * 4), gpu.DeviceBuffer(B * heads * new_len * 4)
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_attention_fwd(dq.ptr, dk.ptr, dv.ptr, out.ptr, dm.ptr, dl.ptr, dtype, B, new_len, total,
                                          heads, hd, dim, dim, dim, dim, float(scale), old_len, causal, status.ptr,
                                          None))
    gpu.sync()
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    return (gpu.download(out, dtype, q.shape), dm.to_numpy(np.float32, (B, heads, new_len)),
            dl.to_numpy(np.float32, (B, heads, new_len)))


@pytest.mark.parametrize("B,S,H,D", [(2, 7, 4, 16), (1, 40, 2, 64), (2, 33, 1, 128), (1, 5, 1, 200)])
def test_cuda_core_attention_matches_oracle(gpu, B, S, H, D):
    rng = np.random.default_rng(B * S + H + D)
    q, k, v = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(3))
    out, m, l = attention(gpu, q, k, v, H, gpu.F32)
    want = O.attention_core(q, k, v, H, exact_order=False)
    assert np.max(np.abs(out - want)) <= 1e-4
    # statistics: row max of scaled scores and sum of exponentials
    sc = np.einsum("bqhd,bkhd->bhqk", q.reshape(B, S, H, D), k.reshape(B, S, H, D)) / np.sqrt(np.float32(D))
    sc = np.where(np.arange(S)[None, None, None, :] > np.arange(S)[None, None, :, None], -np.inf, sc)
    assert np.allclose(m, sc.max(-1), atol=1e-4)
    assert np.allclose(l, np.exp(sc - sc.max(-1, keepdims=True)).sum(-1), rtol=1e-4)


def test_cuda_core_attention_cache_offset_and_bidirectional(gpu):
    rng = np.random.default_rng(21)
    B, H, D, old, new = 2, 2, 32, 5, 4
    k, v = (rng.standard_normal((B, old + new, H * D)).astype(np.float32) for _ in range(2))
    q = rng.standard_normal((B, new, H * D)).astype(np.float32)
    out, _, _ = attention(gpu, q, k, v, H, gpu.F32, old_len=old)
    assert np.max(np.abs(out - O.attention_core(q, k, v, H, old_len=old, exact_order=False))) <= 1e-4
    out, _, _ = attention(gpu, q, k[:, :new], v[:, :new], H, gpu.F32, causal=0)
    assert np.max(np.abs(out - O.attention_core(q, k[:, :new], v[:, :new], H, causal=False, exact_order=False))) <= 1e-4
    # head_dim above the reference's limit is refused
    st = gpu.lib().bfb_attention_fwd(None, None, None, None, None, None, gpu.F32, 1, 2, 2, 1, 300, 300, 300, 300, 300,
                                     1.0, 0, 1, None, None)
    assert st == gpu.INVALID_ARGUMENT


def test_pool_reuses_exact_sizes(gpu):
    lib = gpu.lib()
    p1, p2 = C.c_void_p(), C.c_void_p()
    gpu.check(lib.bfb_pool_acquire(12345, C.byref(p1)))
    lib.bfb_pool_release(p1, 12345)
    gpu.check(lib.bfb_pool_acquire(12345, C.byref(p2)))
    assert p1.value == p2.value
    lib.bfb_pool_release(p2, 12345)
    cached, live = C.c_size_t(), C.c_size_t()
    gpu.check(lib.bfb_pool_stats(C.byref(cached), C.byref(live)))
    assert cached.value >= 12345
    gpu.check(lib.bfb_pool_acquire(0, C.byref(p1)))
    assert p1.value is None


@pytest.mark.parametrize("n,dtype_name", [(8192 * 3 + 77, "f32"), (8192 * 5, "bf16"), (13, "bf16"), (1 << 20, "bf16")])
def test_quantize_e4m3_one_call(gpu, n, dtype_name):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    x[n // 2] = -37.5                                   # the maximum sits in the middle of a chunk
    dtype = gpu.F32 if dtype_name == "f32" else gpu.BF16
    if dtype == gpu.BF16:
        x = O.round_bf16(x)
    src = gpu.upload(x, dtype)
    out = gpu.DeviceBuffer(n)
    scales = gpu.DeviceBuffer.zeros(12)
    winv = gpu.DeviceBuffer.from_numpy(np.array([0.25], np.float32))
    gpu.check(gpu.lib().bfb_quantize_e4m3(src.ptr, dtype, n, out.ptr, scales.ptr, winv.ptr, None))
    s = scales.to_numpy(np.float32, (3,))
    want_scale = np.float32(448.0) / np.float32(37.5)
    assert s[0] == want_scale and s[1] == np.float32(1.0) / want_scale and s[2] == s[1] * np.float32(0.25)
    assert np.array_equal(gpu.download(out, gpu.FP8_E4M3, (n,)), O.e4m3_round_hw(x * want_scale))
    # all-zero tensor: scale 1, zeros out; empty tensor: scales only
    zero = gpu.DeviceBuffer.zeros(64 * 4)
    gpu.check(gpu.lib().bfb_quantize_e4m3(zero.ptr, gpu.F32, 64, out.ptr, scales.ptr, None, None))
    assert scales.to_numpy(np.float32, (3,)).tolist() == [1.0, 1.0, 1.0]
    assert gpu.lib().bfb_quantize_e4m3(None, gpu.F32, 0, None, scales.ptr, None, None) == gpu.OK
    assert gpu.lib().bfb_quantize_e4m3(src.ptr, gpu.FP8_E4M3, n, out.ptr, scales.ptr, None, None) == gpu.INVALID_ARGUMENT


@pytest.mark.parametrize("rows,dim", [(37, 2048), (5, 300), (64, 8192), (3, 8)])
def test_rmsnorm_quantize_e4m3_equals_norm_then_quantize(gpu, rows, dim):
    """The fused call must give what rmsnorm to bf16 followed by bfb_quantize_e4m3 gives: same scale, same codes
    (a last-bit difference in a row's 1/rms may move single values across a rounding boundary)."""
    rng = np.random.default_rng(rows * dim)
    x = O.round_bf16((rng.standard_normal((rows, dim)) * rng.uniform(0.1, 4.0, size=(rows, 1))).astype(np.float32))
    src = gpu.upload(x, gpu.BF16)
    normed = gpu.DeviceBuffer(x.size * 2)
    gpu.check(gpu.lib().bfb_rmsnorm(src.ptr, gpu.BF16, normed.ptr, gpu.BF16, rows, dim, 1e-6, None))
    want_q, want_s = gpu.DeviceBuffer(x.size), gpu.DeviceBuffer.zeros(12)
    winv = gpu.DeviceBuffer.from_numpy(np.array([0.5], np.float32))
    gpu.check(gpu.lib().bfb_quantize_e4m3(normed.ptr, gpu.BF16, x.size, want_q.ptr, want_s.ptr, winv.ptr, None))
    got_q, got_s = gpu.DeviceBuffer(x.size), gpu.DeviceBuffer.zeros(12)
    gpu.check(gpu.lib().bfb_rmsnorm_quantize_e4m3(src.ptr, rows, dim, 1e-6, got_q.ptr, got_s.ptr, winv.ptr, None))
    ws, gs = want_s.to_numpy(np.float32, (3,)), got_s.to_numpy(np.float32, (3,))
    assert np.max(np.abs(ws - gs) / ws) <= 2.0 ** -7            # the maximum may sit one bf16 step apart
    a = gpu.download(want_q, gpu.FP8_E4M3, x.shape)
    b = gpu.download(got_q, gpu.FP8_E4M3, x.shape)
    if np.array_equal(ws, gs):
        assert np.mean(a != b) <= 2e-3 and np.max(np.abs(a - b) / (np.abs(a) + 2.0 ** -6)) <= 0.13
    # against the definition: oracle rmsnorm, rounded to bf16, scaled by this call's scale, rounded to e4m3
    want = O.e4m3_round_hw(O.round_bf16(O.rmsnorm(x)) * gs[0])
    assert np.mean(b != want) <= 2e-3
