"""The numpy restatement (oracle/bf_oracle.py) against the reference: known answers taken from the
statements of the reference's own tests, the committed golden fixtures (outputs of the reference),
and the live reference library when it is present."""
import os
import tempfile

import numpy as np
import pytest

from oracle import bf_oracle as O
from tests.conftest import GOLDEN

C1 = dict(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32)


# ---- known answers (tests/backend/cpu/ops_tests.cpp:36-119, quantize_tests.cpp:12-100) ------------

def test_matmul_known_answer():
    out = O.matmul([[1, 2], [3, 4]], [[5, 6], [7, 8]])
    assert out.tolist() == [[19, 22], [43, 50]]


def test_matmul_rejects_bad_shapes():
    with pytest.raises(O.InvalidArgument):
        O.matmul(np.ones((2, 3)), np.ones((2, 2)))
    with pytest.raises(O.InvalidArgument):
        O.add(np.ones(2), np.ones(3))


def test_linear_identity_weight_plus_bias():
    out = O.linear([[3, 4]], [[1, 0], [0, 1]], [10, 20])
    assert out.tolist() == [[13, 24]]


def test_add_bias_broadcasts_rows():
    out = O.add_bias([[1, 2], [3, 4]], [10, 20])
    assert out.tolist() == [[11, 22], [13, 24]]


def test_activations_limits():
    x = np.array([0.0, 20.0, -20.0], dtype=np.float32)
    for fn in (O.silu, O.gelu):
        y = fn(x)
        assert y[0] == 0 and abs(y[1] - 20) < 0.01 and abs(y[2]) < 0.01
    assert O.relu(np.array([-2.0, 0.0, 3.0])).tolist() == [0, 0, 3]


def test_rmsnorm_unit_rms_and_ratio():
    y = O.rmsnorm(np.array([[1, 2, 3, 4], [-1, -1, -1, -1]], dtype=np.float32))
    assert np.allclose(np.sqrt((y.astype(np.float64) ** 2).mean(axis=1)), 1.0, atol=1e-3)
    z = O.rmsnorm(np.array([[2.0, -4.0]], dtype=np.float32))
    assert z[0, 0] > 0 > z[0, 1] and abs(z[0, 1] / z[0, 0] + 2) < 1e-4
    with pytest.raises(O.InvalidArgument):
        O.rmsnorm(np.ones(4, dtype=np.float32))


def test_softmax_rows_sum_to_one():
    y = O.softmax(np.array([[1, 2, 3], [-1, 0, 1]], dtype=np.float32))
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-5) and (y > 0).all()


def test_embedding_rows_and_range():
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    out = O.embedding_lookup([[0, 2], [3, 1]], table)
    assert out.shape == (2, 2, 3) and out[0, 1].tolist() == [6, 7, 8]
    with pytest.raises(O.InvalidArgument):
        O.embedding_lookup([[4]], table)
    with pytest.raises(O.InvalidArgument):
        O.embedding_lookup([[-1]], table)


def test_positional_broadcast_and_limit():
    x = np.zeros((2, 3, 2), dtype=np.float32)
    pos = np.arange(8, dtype=np.float32).reshape(4, 2)
    out = O.add_positional_embedding(x, pos)
    assert np.array_equal(out[0], pos[:3]) and np.array_equal(out[1], pos[:3])
    assert np.array_equal(O.add_positional_embedding(x, pos, 1)[0], pos[1:4])
    with pytest.raises(O.InvalidArgument):
        O.add_positional_embedding(np.zeros((1, 5, 2), dtype=np.float32), pos)


def test_zero_weights_are_identity_through_residual():
    x = np.random.default_rng(0).standard_normal((2, 5, 8)).astype(np.float32)
    z = np.zeros((8, 8), dtype=np.float32)
    assert np.array_equal(O.self_attention(x, z, z, z, z, 2), x)
    assert np.array_equal(O.feed_forward(x, np.zeros((8, 16)), np.zeros(16), np.zeros((16, 8)), np.zeros(8)), x)


def test_causal_mask_future_token_leaves_past_bit_identical():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 6, 8)).astype(np.float32)
    w = [rng.standard_normal((8, 8)).astype(np.float32) * 0.3 for _ in range(4)]
    y0 = O.self_attention(x, *w, 2)
    x2 = x.copy()
    x2[0, 5] += 1.0
    y1 = O.self_attention(x2, *w, 2)
    assert np.array_equal(y0[0, :5], y1[0, :5]) and not np.array_equal(y0[0, 5], y1[0, 5])


def test_attention_rejects_heads_not_dividing_dim():
    with pytest.raises(O.InvalidArgument):
        O.self_attention(np.zeros((1, 2, 6), dtype=np.float32), *[np.zeros((6, 6))] * 4, 4)


def test_quantize_known_answers():
    assert O.quantize(np.array([1000.0, -1000.0]), "fp8.e4m3").tolist() == [448.0, -448.0]
    assert O.quantize(np.array([1e6, -1e6]), "fp8.e5m2").tolist() == [57344.0, -57344.0]
    x = np.random.default_rng(2).standard_normal(100).astype(np.float32)
    once = O.quantize(x, "bf16")
    assert np.array_equal(O.quantize(once, "bf16"), once)
    special = np.array([np.inf, -np.inf, 0.0], dtype=np.float32)
    for dt in ("bf16", "fp16", "fp8.e4m3", "fp8.e5m2", "tf32"):
        assert np.array_equal(O.quantize(special, dt), special)
    assert np.isnan(O.quantize(np.array([np.nan], dtype=np.float32), "bf16")[0])
    assert np.array_equal(O.quantize(x, "fp32"), x)


def test_hw_e4m3_rounding_matches_simulated_off_ties():
    x = (np.random.default_rng(3).standard_normal(4000) * 40).astype(np.float32)
    x = x[np.abs(x) >= 2.0 ** -6]
    a, b = O.e4m3_round_hw(x), O.quantize(x, "fp8.e4m3")
    # both land on the e4m3 grid; they can differ only at exact ties (never for random inputs)
    assert np.array_equal(a, b)


# ---- golden fixtures: outputs of the reference's CPU backend -------------------------------------------

def _same(a, b, exact, tol=1e-6):
    if exact:
        assert np.array_equal(a, b)
    else:
        assert a.shape == b.shape and np.max(np.abs(a - b) / (1 + np.abs(b))) <= tol


def test_golden_ops(golden_ops):
    g = golden_ops
    x = g["unary_x"]
    _same(O.relu(x), g["unary_relu"], True)
    _same(O.rmsnorm(x), g["unary_rmsnorm"], True)
    _same(O.softmax(x), g["unary_softmax"], False, 1e-7)
    _same(O.silu(x), g["unary_silu"], False)
    _same(O.gelu(x), g["unary_gelu"], False)
    _same(O.matmul(g["mm_a"], g["mm_b"]), g["mm_ab"], True)
    _same(O.matmul_transpose_b(g["mm_a"], g["mm_c"]), g["mm_act"], True)
    _same(O.linear(g["mm_a"].reshape(1, 17, 33), g["mm_b"], g["lin_bias"]), g["lin_out"], True)
    _same(O.add_bias(g["mm_ab"], g["lin_bias"]), g["addbias_out"], True)
    emb = O.embedding_lookup(g["emb_ids"], g["emb_table"])
    _same(emb, g["emb_out"], True)
    _same(O.add_positional_embedding(emb, g["emb_pos"]), g["pos_out"], True)
    _same(O.add_positional_embedding(emb, g["emb_pos"], 2), g["pos_at2_out"], True)
    w = [g["attn_" + n] for n in ("wq", "wk", "wv", "wo")]
    _same(O.self_attention(g["attn_x"], *w, 4), g["attn_out"], False, 1e-6)
    _same(O.feed_forward(g["attn_x"], g["ff_w1"], g["ff_b1"], g["ff_w2"], g["ff_b2"]), g["ff_out"], False, 1e-6)
    for dt in ("bf16", "fp16", "tf32", "fp8.e4m3", "fp8.e5m2"):
        _same(O.quantize(g["q_x"], dt), g["q_" + dt.replace(".", "_")], True)


def test_golden_c1_checkpoint_route(golden_c1_normal):
    g = golden_c1_normal
    ops = O.lm_ops(**C1)
    params = O.synth_params(ops, None, seed=int(g["seed"][0]), sigma=0.02)
    ids = O.synth_token_ids(4, 32, 256, seed=int(g["seed"][1]))
    assert np.array_equal(ids, g["ids"])
    logits = O.model_forward(ops, params, ids)
    assert np.max(np.abs(logits - g["logits"])) <= 1e-6
    cpu_bf16 = O.model_forward(ops, params, ids, cpu_policy={"storage": "bf16", "compute": "bf16"})
    assert np.max(np.abs(cpu_bf16 - g["logits_cpu_bf16"])) <= 1e-6


def test_checkpoint_round_trip_and_errors():
    ops = O.lm_ops(vocab=8, dim=8, layers=1, heads=2, hidden=16, max_seq=6)
    params = O.synth_params(ops, None, seed=3, sigma=0.1)
    with tempfile.TemporaryDirectory() as tmp:
        p = os.path.join(tmp, "a.bfckpt")
        O.save_checkpoint(p, list(params.items()))
        raw = open(p, "rb").read()
        assert raw[:8] == b"BFCKPT1\x00" and int.from_bytes(raw[8:12], "little") == len(params)
        back = O.load_checkpoint(p)
        assert [n for n, _ in back] == list(params) and all(np.array_equal(v, params[n]) for n, v in back)
        with pytest.raises(O.RuntimeFailure):
            O.load_checkpoint(os.path.join(tmp, "missing.bfckpt"))
        open(p, "wb").write(b"NOTACKPT" + raw[8:])
        with pytest.raises(O.RuntimeFailure):
            O.load_checkpoint(p)
        open(p, "wb").write(raw[:-5])
        with pytest.raises(O.RuntimeFailure):
            O.load_checkpoint(p)


def test_param_layout_names_follow_value_ids():
    ops = O.lm_ops(vocab=6, dim=4, layers=1, heads=2, hidden=8, max_seq=4)
    names = [n for n, _ in O.param_layout(ops)]
    assert names == ["embedding1.table", "positional_embedding2.table", "attention3.wq", "attention3.wk",
                     "attention3.wv", "attention3.wout", "feedforward4.w1", "feedforward4.b1", "feedforward4.w2",
                     "feedforward4.b2", "linear5.weight", "linear5.bias"]


# ---- live reference (only where oracle/_ref was built) ---------------------------------------------------

def test_live_reference_agrees(ref):
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal((9, 20)).astype(np.float32), rng.standard_normal((20, 11)).astype(np.float32)
    assert np.array_equal(ref.matmul(a, b), O.matmul(a, b))
    x = rng.standard_normal((4, 3, 50)).astype(np.float32)
    assert np.array_equal(ref.rmsnorm(x), O.rmsnorm(x))
    assert np.allclose(ref.softmax(x), O.softmax(x), atol=1e-7)
    src = O.lm_source(seq=32, **C1)
    compiled = ref.Compiled(src)
    assert compiled.ops() == O.lm_ops(**C1)
    model = ref.Model(compiled, 42)
    names = model.param_names()
    assert names == [n for n, _ in O.param_layout(compiled.ops())]
    params = {n: model.param(i) for i, n in enumerate(names)}
    ids = compiled.synthetic_input(42, 2)
    assert np.max(np.abs(model.forward(ids) - O.model_forward(compiled.ops(), params, ids))) <= 1e-6
    with pytest.raises(ref.RefError) as e:
        ref.matmul(np.ones((2, 3)), np.ones((2, 2)))
    assert e.value.kind == "invalid_argument"


def test_live_reference_precision_block_parses(ref):
    src = O.lm_source(seq=8, vocab=16, dim=8, layers=1, heads=2, hidden=16, max_seq=8,
                      precision={"storage": "bf16", "compute": "fp8.e4m3", "accumulate": "fp32"})
    assert ref.Compiled(src).precision() == {"storage": "bf16", "compute": "fp8.e4m3", "accumulate": "fp32"}


# ---- attention backward (src/backend/cuda/fused_attention.cu:158-380) ------------------------------------------

def _attention_loss64(q, k, v, g, heads, scale, old_len):
    """sum(dOut * attention(q, k, v)) in float64, written independently of the oracle's backward."""
    B, new_len, dim = q.shape
    total, hd = k.shape[1], dim // heads
    loss = 0.0
    i = np.arange(new_len)[:, None]
    j = np.arange(total)[None, :]
    for b in range(B):
        for h in range(heads):
            sl = slice(h * hd, (h + 1) * hd)
            s = (q[b, :, sl] @ k[b, :, sl].T) * scale
            s = np.where(j > old_len + i, -np.inf, s)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            loss += float(((p @ v[b, :, sl]) * g[b, :, sl]).sum())
    return loss


def test_attention_backward_matches_finite_differences():
    rng = np.random.default_rng(77)
    B, H, D, old, new = 1, 2, 4, 2, 5
    q, g = (rng.standard_normal((B, new, H * D)) for _ in range(2))
    k, v = (rng.standard_normal((B, old + new, H * D)) for _ in range(2))
    scale = 0.5
    out, m, l = O.attention_forward_stats(q, k, v, H, scale, old)
    dq, dk, dv = O.attention_backward(g, q, k, v, out, m, l, H, scale, old)
    eps = 1e-5
    for name, x, grad in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        num = np.zeros_like(x)
        for idx in np.ndindex(*x.shape):
            keep = x[idx]
            x[idx] = keep + eps
            up = _attention_loss64(q, k, v, g, H, scale, old)
            x[idx] = keep - eps
            down = _attention_loss64(q, k, v, g, H, scale, old)
            x[idx] = keep
            num[idx] = (up - down) / (2 * eps)
        # the oracle takes fp32 operands and fp32 (out, m, l): 1e-5 relative
        assert np.max(np.abs(num - grad)) <= 2e-5 * max(1.0, np.max(np.abs(num))), name


def test_attention_backward_matches_the_reference_kernel_outputs():
    """Outputs of the reference's own fusedAttentionForward + fusedAttentionBackward, produced on a B200 by
    tests/golden/make_attention_backward_golden.py: the oracle's forward statistics and its gradients agree with them
    to fp32 rounding."""
    gold = dict(np.load(os.path.join(GOLDEN, "attention_backward.npz")))
    for tag in ("small", "hd128"):
        heads, old = int(gold[f"{tag}_heads"]), int(gold[f"{tag}_old_len"])
        g, q, k, v = (gold[f"{tag}_{n}"] for n in ("d_out", "q", "k", "v"))
        scale = float(1.0 / np.sqrt(np.float32(q.shape[2] // heads)))
        out, m, l = O.attention_forward_stats(q, k, v, heads, scale, old)
        assert np.max(np.abs(out - gold[f"{tag}_out"])) <= 1e-5
        # the reference keeps a running maximum: m is the final maximum either way, l the matching sum
        assert np.allclose(m, gold[f"{tag}_m"], atol=1e-5) and np.allclose(l, gold[f"{tag}_l"], rtol=1e-5)
        got = O.attention_backward(g, q, k, v, gold[f"{tag}_out"], gold[f"{tag}_m"], gold[f"{tag}_l"], heads, scale, old)
        for name, a in zip(("dq", "dk", "dv"), got):
            want = gold[f"{tag}_{name}"]
            assert np.max(np.abs(a - want)) <= 2e-5 * max(1.0, float(np.max(np.abs(want)))), (tag, name)
