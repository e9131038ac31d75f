"""GPU parity of the attention core's backward (bfb_attention_bwd) through the C ABI: the CUDA-core kernel in fp32 and
the tcgen05 kernel (head_dim 128, bf16 operands), against the oracle's float64 restatement of fusedAttentionBackward
(src/backend/cuda/fused_attention.cu:158-380), against the committed outputs of the reference's own kernel, and
against that kernel run on the same GPU when oracle/_ref/libbf_ref_cuda.so is present."""
import os

import numpy as np
import pytest

from oracle import bf_oracle as O
from tests.conftest import GOLDEN

pytestmark = pytest.mark.gpu

# fp32 route: fp32 dot products and atomics against float64
TOL_F32 = 2e-4
# bf16 route: probabilities and dS rounded to bf16 (2^-9 relative each) and summed over up to thousands of rows,
# relative to the largest gradient entry
TOL_BF16 = 1.0e-2


def attention_backward(gpu, d_out, q, k, v, out, m, l, heads, dtype, old_len=0, causal=1, scale=None):
    B, new_len, dim = q.shape
    total = k.shape[1]
    hd = dim // heads
    scale = 1.0 / np.sqrt(np.float32(hd)) if scale is None else scale
    d_g, d_q, d_k, d_v, d_o = (gpu.upload(t, dtype) for t in (d_out, q, k, v, out))
    d_m, d_l = gpu.upload(np.ascontiguousarray(m, np.float32), gpu.F32), gpu.upload(np.ascontiguousarray(l, np.float32), gpu.F32)
    # results start as NaN: every element must be written
    nan_q = np.full((B, new_len, dim), np.nan, np.float32)
    nan_k = np.full((B, total, dim), np.nan, np.float32)
    g_q, g_k, g_v = gpu.upload(nan_q, gpu.F32), gpu.upload(nan_k, gpu.F32), gpu.upload(nan_k, gpu.F32)
    scratch = gpu.DeviceBuffer(max(1, 2 * B * heads * new_len) * 4)
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_attention_bwd(d_g.ptr, d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, d_m.ptr, d_l.ptr, g_q.ptr, g_k.ptr,
                                          g_v.ptr, scratch.ptr, dtype, B, new_len, total, heads, hd, dim, dim, dim, dim,
                                          float(scale), old_len, causal, status.ptr, None))
    gpu.sync()
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    return (gpu.download(g_q, gpu.F32, (B, new_len, dim)), gpu.download(g_k, gpu.F32, (B, total, dim)),
            gpu.download(g_v, gpu.F32, (B, total, dim)))


def case(rng, B, new_len, total, H, D, bf16, spread=1.0):
    r = O.round_bf16 if bf16 else (lambda x: x)
    q = r(rng.standard_normal((B, new_len, H * D)).astype(np.float32) * spread)
    k = r(rng.standard_normal((B, total, H * D)).astype(np.float32) * spread)
    v = r(rng.standard_normal((B, total, H * D)).astype(np.float32))
    g = r(rng.standard_normal((B, new_len, H * D)).astype(np.float32))
    scale = float(1.0 / np.sqrt(np.float32(D)))
    out, m, l = O.attention_forward_stats(q, k, v, H, scale, total - new_len)
    return g, q, k, v, r(out), m, l, scale


def close(got, want, tol):
    assert np.isfinite(got).all()
    bound = tol * max(1.0, float(np.max(np.abs(want))))
    return float(np.max(np.abs(got - want))) <= bound


@pytest.mark.parametrize("B,S,H,D", [(2, 7, 4, 16), (1, 40, 2, 64), (2, 33, 1, 128), (1, 5, 1, 200), (1, 1, 1, 8)])
def test_cuda_core_backward_matches_oracle(gpu, B, S, H, D):
    rng = np.random.default_rng(7 * B + S + H + D)
    g, q, k, v, out, m, l, scale = case(rng, B, S, S, H, D, False)
    want = O.attention_backward(g, q, k, v, out, m, l, H, scale)
    got = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.F32)
    for a, b in zip(got, want):
        assert close(a, b, TOL_F32)


def test_cuda_core_backward_with_cached_keys(gpu):
    rng = np.random.default_rng(41)
    B, H, D, old, new = 2, 2, 32, 13, 9
    g, q, k, v, out, m, l, scale = case(rng, B, new, old + new, H, D, False)
    want = O.attention_backward(g, q, k, v, out, m, l, H, scale, old)
    got = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.F32, old_len=old)
    for a, b in zip(got, want):
        assert close(a, b, TOL_F32)


@pytest.mark.parametrize("B,S,H", [(1, 128, 1), (2, 256, 2), (1, 384, 1), (1, 200, 2), (3, 50, 1), (1, 1, 1), (1, 1000, 1)])
def test_tensor_core_backward_matches_oracle(gpu, B, S, H):
    rng = np.random.default_rng(B * 1000 + S + H)
    g, q, k, v, out, m, l, scale = case(rng, B, S, S, H, 128, True)
    want = O.attention_backward(g, q, k, v, out, m, l, H, scale)
    got = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.BF16)
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert close(a, b, TOL_BF16), name


def test_tensor_core_backward_with_cached_keys_and_peaked_scores(gpu):
    rng = np.random.default_rng(42)
    B, H, old, new = 2, 2, 200, 150
    g, q, k, v, out, m, l, scale = case(rng, B, new, old + new, H, 128, True)
    want = O.attention_backward(g, q, k, v, out, m, l, H, scale, old)
    got = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.BF16, old_len=old)
    for a, b in zip(got, want):
        assert close(a, b, TOL_BF16)
    # scaled scores of a few tens: probabilities near one-hot, exponentials of masked entries must not leak
    g, q, k, v, out, m, l, scale = case(rng, 1, 256, 256, 1, 128, True, spread=3.0)
    want = O.attention_backward(g, q, k, v, out, m, l, 1, scale)
    got = attention_backward(gpu, g, q, k, v, out, m, l, 1, gpu.BF16)
    for a, b in zip(got, want):
        assert close(a, b, 2 * TOL_BF16)


def test_backward_empty_and_rejected_inputs(gpu):
    z = np.zeros((0, 4, 128), np.float32)
    st = np.zeros((0, 1, 4), np.float32)
    got = attention_backward(gpu, z, z, z, z, z, st, st, 1, gpu.BF16)
    assert all(t.size == 0 for t in got)
    code = gpu.lib().bfb_attention_bwd(None, None, None, None, None, None, None, None, None, None, None, gpu.F32, 1, 2, 2,
                                       1, 300, 300, 300, 300, 300, 1.0, 0, 1, None, None)
    assert code == gpu.INVALID_ARGUMENT
    # valid sizes with a missing operand: refused on the host, nothing is launched
    buf = gpu.DeviceBuffer.zeros(2 * 2 * 16 * 4)
    code = gpu.lib().bfb_attention_bwd(buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, None, buf.ptr, buf.ptr, buf.ptr,
                                       buf.ptr, gpu.F32, 1, 2, 2, 1, 16, 16, 16, 16, 16, 1.0, 0, 1, None, None)
    assert code == gpu.INVALID_ARGUMENT and b"null" in gpu.lib().bfb_last_error()
    # a row stride below heads * head_dim
    code = gpu.lib().bfb_attention_bwd(buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr,
                                       buf.ptr, gpu.F32, 1, 2, 2, 1, 16, 8, 16, 16, 16, 1.0, 0, 1, None, None)
    assert code == gpu.INVALID_ARGUMENT


def test_backward_against_committed_reference_outputs(gpu):
    """The reference's own fusedAttentionForward + fusedAttentionBackward outputs (fp32, produced on a B200 by
    tests/golden/make_attention_backward_golden.py) for both routes."""
    path = os.path.join(GOLDEN, "attention_backward.npz")
    gold = dict(np.load(path))
    for tag, dtype, tol in (("small", gpu.F32, TOL_F32), ("hd128", gpu.BF16, TOL_BF16)):
        heads, old = int(gold[f"{tag}_heads"]), int(gold[f"{tag}_old_len"])
        g, q, k, v = (gold[f"{tag}_{n}"] for n in ("d_out", "q", "k", "v"))
        out, m, l = gold[f"{tag}_out"], gold[f"{tag}_m"], gold[f"{tag}_l"]
        if dtype == gpu.BF16:
            out = O.round_bf16(out)    # the inputs of this case are bf16-valued already
        scale = float(1.0 / np.sqrt(np.float32(q.shape[2] // heads)))
        got = attention_backward(gpu, g, q, k, v, out, m, l, heads, dtype, old_len=old)
        for name, a in zip(("dq", "dk", "dv"), got):
            assert close(a, gold[f"{tag}_{name}"], tol), (tag, name)


@pytest.fixture(scope="module")
def refcuda():
    from oracle import ref_lib
    if not ref_lib.cuda_available():
        pytest.skip("oracle/_ref/libbf_ref_cuda.so not built")
    return ref_lib


@pytest.mark.parametrize("old_len", [0, 96])
def test_backward_against_the_reference_kernel_on_this_gpu(gpu, refcuda, old_len):
    """Both routes against fusedAttentionBackward of the reference (compiled unmodified) on the same inputs, with the
    reference's own forward output and row statistics as the operands."""
    rng = np.random.default_rng(50 + old_len)
    B, H, D, new = 2, 4, 128, 320
    g, q, k, v, _, _, _, scale = case(rng, B, new, old_len + new, H, D, True)
    want = refcuda.cuda_fused_attention_backward(g, q, k, v, H, scale, old_len)
    for dtype, tol in ((gpu.F32, TOL_F32), (gpu.BF16, TOL_BF16)):
        out = O.round_bf16(want["out"]) if dtype == gpu.BF16 else want["out"]
        got = attention_backward(gpu, g, q, k, v, out, want["m"], want["l"], H, dtype, old_len=old_len)
        for name, a in zip(("dq", "dk", "dv"), got):
            print(f"attention backward dtype {dtype} {name}: max abs diff", float(np.max(np.abs(a - want[name]))),
                  "of", float(np.max(np.abs(want[name]))))
            assert close(a, want[name], tol), (dtype, name)


def test_full_size_properties(gpu):
    """At the attention benchmark's per-head shape (sequence 2048, head_dim 128), properties that need no oracle run:
    the gradients are linear in dOut (exactly, for a power-of-two factor, where one CTA owns the sum), keys that are
    all equal give dQ = 0 (the rows of dS sum to zero), and a leading slice is a closed problem (causality)."""
    S, H = 2048, 2
    rng = np.random.default_rng(60)
    g, q, k, v, out, m, l, scale = case(rng, 1, S, S, H, 128, True)
    a = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.BF16)
    b = attention_backward(gpu, 4.0 * g, q, k, v, out, m, l, H, gpu.BF16)
    # dQ is summed with atomics in an order that varies: linear up to fp32 rounding; dK and dV exactly
    assert np.array_equal(4.0 * a[1], b[1]) and np.array_equal(4.0 * a[2], b[2])
    assert np.max(np.abs(4.0 * a[0] - b[0])) <= 1e-5 * np.max(np.abs(b[0]))
    k_same = np.broadcast_to(k[:, :1, :], k.shape).copy()
    out2, m2, l2 = O.attention_forward_stats(q[:, :256], k_same[:, :256], v[:, :256], H, scale, 0)
    dq, _, _ = attention_backward(gpu, g[:, :256], q[:, :256], k_same[:, :256], v[:, :256], O.round_bf16(out2), m2, l2, H,
                                  gpu.BF16)
    assert np.max(np.abs(dq)) <= 2e-2 * np.max(np.abs(a[0]))
    # sampled rows of the full-size result against the oracle on a leading slice (causality: the first 256 queries and
    # keys form a closed problem for dQ)
    want = O.attention_backward(g[:, :256], q[:, :256], k[:, :256], v[:, :256], out[:, :256], m[:, :, :256], l[:, :, :256],
                                H, scale)
    assert close(a[0][:, :256], want[0], TOL_BF16)


# ---- gradients of C = A B on the bf16 route (matmulBf16Backward, src/backend/cuda/ops_tensorcore.cu:389-417) ----------

def matmul_bf16_backward(gpu, a, b, grad):
    (m, k), n = a.shape, b.shape[1]
    d_a, d_b, d_g = (gpu.upload(t, gpu.F32) for t in (a, b, grad))
    out_a = gpu.upload(np.full((m, k), np.nan, np.float32), gpu.F32)
    out_b = gpu.upload(np.full((k, n), np.nan, np.float32), gpu.F32)
    gpu.check(gpu.lib().bfb_matmul_bf16_backward(d_a.ptr, d_b.ptr, d_g.ptr, out_a.ptr, out_b.ptr, m, k, n, None))
    gpu.sync()
    return gpu.download(out_a, gpu.F32, (m, k)), gpu.download(out_b, gpu.F32, (k, n))


@pytest.mark.parametrize("m,k,n", [(256, 512, 384), (300, 136, 200), (33, 37, 21), (1, 8, 8), (2048, 1024, 256)])
def test_matmul_bf16_backward_matches_oracle(gpu, m, k, n):
    """Tensor-core sizes, ragged sizes (odd leading dimensions go to the CUDA-core kernel) and a single row."""
    rng = np.random.default_rng(m + k + n)
    a, b, g = (rng.standard_normal(s).astype(np.float32) for s in ((m, k), (k, n), (m, n)))
    a16, b16, g16 = O.round_bf16(a), O.round_bf16(b), O.round_bf16(g)
    want_a = g16.astype(np.float64) @ b16.astype(np.float64).T
    want_b = a16.astype(np.float64).T @ g16.astype(np.float64)
    got_a, got_b = matmul_bf16_backward(gpu, a, b, g)
    # exact products of bf16 values, fp32 accumulation
    assert close(got_a, want_a, 2e-5) and close(got_b, want_b, 2e-5)


def test_matmul_bf16_backward_zero_dimension_zero_fills(gpu):
    a, b, g = np.zeros((4, 0), np.float32), np.zeros((0, 3), np.float32), np.ones((4, 3), np.float32)
    got_a, got_b = matmul_bf16_backward(gpu, a, b, g)
    assert got_a.shape == (4, 0) and got_b.shape == (0, 3)
    a, b, g = np.ones((0, 5), np.float32), np.ones((5, 3), np.float32), np.ones((0, 3), np.float32)
    got_a, got_b = matmul_bf16_backward(gpu, a, b, g)
    assert got_a.shape == (0, 5) and np.array_equal(got_b, np.zeros((5, 3), np.float32))


def test_matmul_bf16_backward_against_the_reference_cublaslt_path(gpu, refcuda):
    rng = np.random.default_rng(71)
    m, k, n = 512, 768, 640
    a, b, g = (rng.standard_normal(s).astype(np.float32) for s in ((m, k), (k, n), (m, n)))
    want_a, want_b = refcuda.cuda_matmul_bf16_backward(a, b, g)
    got_a, got_b = matmul_bf16_backward(gpu, a, b, g)
    print("matmul bf16 backward vs reference: dA", float(np.max(np.abs(got_a - want_a))), "dB", float(np.max(np.abs(got_b - want_b))))
    assert close(got_a, want_a, 2e-5) and close(got_b, want_b, 2e-5)


def test_backward_configuration_2_in_full_against_the_reference_kernel(gpu, refcuda):
    """The attention benchmark's full size (batch 16, 16 heads of 128, sequence 2048, causal): every element of dQ, dK
    and dV from the tensor-core kernel against the reference's fusedAttentionBackward on the same bf16-valued inputs
    (operands: the reference's own forward output and row statistics), and both device times."""
    rng = np.random.default_rng(3)
    B, H, D, S = 16, 16, 128, 2048
    q, k, v, g = (O.round_bf16(rng.standard_normal((B, S, H * D), dtype=np.float32)) for _ in range(4))
    scale = float(D ** -0.5)
    want = refcuda.cuda_fused_attention_backward(g, q, k, v, H, scale, 0, iters=1)
    dim = H * D
    dev = [gpu.upload(t, gpu.BF16) for t in (g, q, k, v, O.round_bf16(want["out"]))]
    d_m, d_l = gpu.upload(want["m"], gpu.F32), gpu.upload(want["l"], gpu.F32)
    grads = [gpu.DeviceBuffer(q.size * 4) for _ in range(3)]
    scratch, status = gpu.DeviceBuffer(B * H * S * 8), gpu.DeviceBuffer.zeros(4)

    def run():
        gpu.check(gpu.lib().bfb_attention_bwd(dev[0].ptr, dev[1].ptr, dev[2].ptr, dev[3].ptr, dev[4].ptr, d_m.ptr, d_l.ptr,
                                              grads[0].ptr, grads[1].ptr, grads[2].ptr, scratch.ptr, gpu.BF16, B, S, S, H, D,
                                              dim, dim, dim, dim, scale, 0, 1, status.ptr, None))
    import torch
    run()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        run()
    b.record()
    torch.cuda.synchronize()
    ours_ms = a.elapsed_time(b) / 3
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    flops = 10.0 * D * B * H * S * (S + 1) / 2.0
    print(f"configuration 2 backward: reference {want['ms']:.1f} ms ({flops / want['ms'] / 1e9:.2f} TFLOP/s causal), "
          f"this kernel {ours_ms:.3f} ms ({flops / ours_ms / 1e9:.1f} TFLOP/s)")
    for name, buf in zip(("dq", "dk", "dv"), grads):
        got = gpu.download(buf, gpu.F32, q.shape)
        err, top = float(np.max(np.abs(got - want[name]))), float(np.max(np.abs(want[name])))
        print(f"  {name}: max abs diff {err:.3e} of {top:.3f}")
        assert np.isfinite(got).all() and err <= TOL_BF16 * max(1.0, top), name


@pytest.mark.parametrize("B,H,old,new,causal", [
    (1, 1, 130, 1, 1),      # one new row after a cache: a single step on every key block
    (1, 3, 0, 129, 1),      # one row into the second query block
    (2, 1, 5, 640, 1),      # five and six steps per key block: both parities of every barrier several times over
    (1, 2, 257, 255, 1),    # cache and rows both off the tile grid
    (1, 1, 0, 300, 0),      # bidirectional: every key block walks every query block
    (1, 2, 64, 64, 0),
])
def test_tensor_core_backward_shapes_off_the_tile_grid(gpu, B, H, old, new, causal):
    rng = np.random.default_rng(B + 10 * H + old + 3 * new + causal)
    D = 128
    r = O.round_bf16
    q = r(rng.standard_normal((B, new, H * D)).astype(np.float32))
    k = r(rng.standard_normal((B, old + new, H * D)).astype(np.float32))
    v = r(rng.standard_normal((B, old + new, H * D)).astype(np.float32))
    g = r(rng.standard_normal((B, new, H * D)).astype(np.float32))
    scale = float(D ** -0.5)
    if causal:
        out, m, l = O.attention_forward_stats(q, k, v, H, scale, old)
        want = O.attention_backward(g, q, k, v, out, m, l, H, scale, old)
    else:
        # every key visible: the oracle's mask j <= old_len + i with old_len = total_len lets everything through
        out, m, l = O.attention_forward_stats(q, k, v, H, scale, old + new)
        want = O.attention_backward(g, q, k, v, out, m, l, H, scale, old + new)
    got = attention_backward(gpu, g, q, k, v, r(out), m, l, H, gpu.BF16, old_len=old, causal=causal)
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert close(a, b, TOL_BF16), name
    # the fp32 route on the same problem
    got32 = attention_backward(gpu, g, q, k, v, out, m, l, H, gpu.F32, old_len=old, causal=causal)
    for name, a, b in zip(("dQ", "dK", "dV"), got32, want):
        assert close(a, b, TOL_F32), name
