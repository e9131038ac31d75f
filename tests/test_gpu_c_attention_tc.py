"""GPU parity of the tcgen05 flash-attention kernel (head_dim 128, bf16 data) through the C ABI,
against the oracle's float64 attention on the same bf16-rounded inputs."""
import numpy as np
import pytest

from oracle import bf_oracle as O
from tests.test_gpu_a_ops import attention

pytestmark = pytest.mark.gpu

# bf16 probabilities and a bf16 result: 2^-8 relative on O(1) values
TOL = 1.2e-2


def qkv(rng, B, new_len, total, H, D=128, scale=1.0):
    q = O.round_bf16(rng.standard_normal((B, new_len, H * D)).astype(np.float32) * scale)
    k = O.round_bf16(rng.standard_normal((B, total, H * D)).astype(np.float32) * scale)
    v = O.round_bf16(rng.standard_normal((B, total, H * D)).astype(np.float32))
    return q, k, v


@pytest.mark.parametrize("B,S,H", [(1, 128, 1), (2, 256, 2), (1, 384, 1), (1, 200, 2), (3, 50, 1), (1, 1, 1)])
def test_causal_prefill_matches_oracle(gpu, B, S, H):
    rng = np.random.default_rng(B * 1000 + S + H)
    q, k, v = qkv(rng, B, S, S, H)
    out, m, l = attention(gpu, q, k, v, H, gpu.BF16)
    want = O.attention_core(q, k, v, H, exact_order=False)
    assert np.max(np.abs(out - want)) <= TOL
    D = 128
    sc = np.einsum("bqhd,bkhd->bhqk", q.reshape(B, S, H, D), k.reshape(B, S, H, D)).astype(np.float64) / np.sqrt(D)
    sc = np.where(np.arange(S)[None, None, None, :] > np.arange(S)[None, None, :, None], -np.inf, sc)
    assert np.allclose(m, sc.max(-1), atol=2e-3)
    assert np.allclose(l, np.exp(sc - sc.max(-1, keepdims=True)).sum(-1), rtol=2e-3)


def test_cache_offset_and_bidirectional(gpu):
    rng = np.random.default_rng(31)
    B, H, old, new = 2, 2, 200, 150
    q, k, v = qkv(rng, B, new, old + new, H)
    out, _, _ = attention(gpu, q, k, v, H, gpu.BF16, old_len=old)
    assert np.max(np.abs(out - O.attention_core(q, k, v, H, old_len=old, exact_order=False))) <= TOL
    q2, k2, v2 = qkv(rng, 1, 130, 130, 1)
    out, _, _ = attention(gpu, q2, k2, v2, 1, gpu.BF16, causal=0)
    assert np.max(np.abs(out - O.attention_core(q2, k2, v2, 1, causal=False, exact_order=False))) <= TOL


def test_large_scores_stay_finite(gpu):
    rng = np.random.default_rng(32)
    q, k, v = qkv(rng, 1, 256, 256, 1, scale=6.0)     # scaled scores of a few hundred: exp must not overflow
    out, _, _ = attention(gpu, q, k, v, 1, gpu.BF16)
    assert np.isfinite(out).all()
    assert np.max(np.abs(out - O.attention_core(q, k, v, 1, exact_order=False))) <= 2 * TOL


def test_causality_future_keys_do_not_change_past_rows(gpu):
    rng = np.random.default_rng(33)
    q, k, v = qkv(rng, 1, 300, 300, 2)
    out0, _, _ = attention(gpu, q, k, v, 2, gpu.BF16)
    k2, v2 = k.copy(), v.copy()
    k2[0, 257:] += 1.0
    v2[0, 257:] -= 2.0
    out1, _, _ = attention(gpu, q, k2, v2, 2, gpu.BF16)
    assert np.array_equal(out0[0, :257], out1[0, :257]) and not np.array_equal(out0[0, 257:], out1[0, 257:])


def test_uniform_values_give_value_mean(gpu):
    # full-size row property (config-2 shape per head): with V constant along keys the output equals it
    S, H = 2048, 2
    rng = np.random.default_rng(34)
    q, k, _ = qkv(rng, 1, S, S, H)
    v = np.broadcast_to(O.round_bf16(rng.standard_normal((1, 1, H * 128)).astype(np.float32)), (1, S, H * 128)).copy()
    out, _, l = attention(gpu, q, k, v, H, gpu.BF16)
    assert np.max(np.abs(out - v)) <= TOL and (l >= 1.0 - 1e-3).all()


def test_interleaved_qkv_strides(gpu):
    # Q, K, V read in place from one [tokens, 3*dim] projection output
    rng = np.random.default_rng(35)
    B, S, H, D = 2, 160, 2, 128
    dim = H * D
    packed = O.round_bf16(rng.standard_normal((B, S, 3 * dim)).astype(np.float32))
    dev = gpu.upload(packed, gpu.BF16)
    out = gpu.DeviceBuffer(B * S * dim * 2)
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_attention_fwd(dev.ptr, dev.ptr + dim * 2, dev.ptr + 2 * dim * 2, out.ptr, None, None,
                                          gpu.BF16, B, S, S, H, D, 3 * dim, 3 * dim, 3 * dim, dim,
                                          float(1 / np.sqrt(D)), 0, 1, status.ptr, None))
    gpu.sync()
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    got = gpu.download(out, gpu.BF16, (B, S, dim))
    q, k, v = packed[..., :dim], packed[..., dim:2 * dim], packed[..., 2 * dim:]
    assert np.max(np.abs(got - O.attention_core(q, k, v, H, exact_order=False))) <= TOL


@pytest.mark.parametrize("B,H,total", [(3, 2, 700), (1, 1, 5000), (2, 16, 1), (5, 3, 263)])
def test_one_query_against_a_cache(gpu, B, H, total):
    """A generation step: one new query per sequence and head against `total` cached keys (the bandwidth-oriented
    kernel, with the keys split over several CTAs when they are many), against the oracle."""
    rng = np.random.default_rng(B * 100 + H * 10 + total)
    q, k, v = qkv(rng, B, 1, total, H)
    out, m, l = attention(gpu, q, k, v, H, gpu.BF16, old_len=total - 1)
    want = O.attention_core(q, k, v, H, old_len=total - 1, exact_order=False)
    assert np.max(np.abs(out - want)) <= TOL
    D = 128
    sc = np.einsum("bqhd,bkhd->bhqk", q.reshape(B, 1, H, D), k.reshape(B, total, H, D)).astype(np.float64) / np.sqrt(D)
    assert np.allclose(m, sc.max(-1), atol=2e-3)
    assert np.allclose(l, np.exp(sc - sc.max(-1, keepdims=True)).sum(-1), rtol=2e-3)
    # bidirectional with one query is the same computation
    out2, _, _ = attention(gpu, q, k, v, H, gpu.BF16, causal=0)
    assert np.array_equal(out, out2)


@pytest.mark.parametrize("B,new,old,H", [(2, 256, 0, 2), (1, 200, 72, 3), (1, 1000, 0, 1)])
def test_output_maxima_for_an_e4m3_quantisation(gpu, B, new, old, H):
    """The epilogue's per-32-row maxima are exactly the maxima of the bf16 output it stores (ragged last blocks and
    cached keys included), and the output itself is what the plain call gives."""
    rng = np.random.default_rng(B + new + old + H)
    q, k, v = qkv(rng, B, new, old + new, H)
    dim = H * 128
    d_q, d_k, d_v = (gpu.upload(t, gpu.BF16) for t in (q, k, v))
    out = gpu.DeviceBuffer(q.size * 2)
    blocks = (new + 127) // 128
    count = B * H * blocks * 4
    maxima = gpu.upload(np.full(count, np.nan, np.float32), gpu.F32)
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_attention_fwd_maxima(d_q.ptr, d_k.ptr, d_v.ptr, out.ptr, maxima.ptr, count, B, new, old + new, H,
                                                 dim, dim, dim, dim, float(1 / np.sqrt(128.0)), old, status.ptr, None))
    gpu.sync()
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    got = gpu.download(out, gpu.BF16, q.shape)
    plain, _, _ = attention(gpu, q, k, v, H, gpu.BF16, old_len=old)
    assert np.array_equal(got, plain)
    padded = np.zeros((B, blocks * 128, H, 128), np.float32)
    padded[:, :new] = np.abs(got).reshape(B, new, H, 128)
    want = padded.reshape(B, blocks, 4, 32, H, 128).max(axis=(3, 5)).transpose(0, 3, 1, 2)      # [B, H, blocks, 4]
    assert np.array_equal(gpu.download(maxima, gpu.F32, (B, H, blocks, 4)), want)
    # one query row has no tensor-core route: refused, not silently without maxima
    code = gpu.lib().bfb_attention_fwd_maxima(d_q.ptr, d_k.ptr, d_v.ptr, out.ptr, maxima.ptr, B * H * 4, B, 1, old + new, H,
                                              dim, dim, dim, dim, 0.1, old + new - 1, status.ptr, None)
    assert code == gpu.UNSUPPORTED
