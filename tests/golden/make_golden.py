"""Generates the golden fixtures in this directory from the REFERENCE ITSELF.

Run where the reference sources exist (oracle/_ref/libbf_ref.so built by `make -C oracle`):

    python tests/golden/make_golden.py

Every expected value below is produced by blackforge::backend::cpu code (through oracle/ref_lib.py);
inputs come from seeded generators. The fixtures pin the numpy restatement (tests/test_oracle.py) and
the GPU kernels (tests/test_gpu_*.py) on machines where the reference library is absent.
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import bf_oracle as O  # noqa: E402
from oracle import ref_lib as R  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# config 1: tiny decoder-only LM, fp32
C1 = dict(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32)
C1_BATCH, C1_SEQ = 4, 32


def ops_fixture():
    rng = np.random.Generator(np.random.PCG64(20240501))
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    out = {}
    x = f(3, 5, 300, scale=3.0)
    out["unary_x"] = x
    for name in ("silu", "relu", "gelu", "rmsnorm", "softmax"):
        out[f"unary_{name}"] = getattr(R, name)(x)
    a, b, c = f(17, 33), f(33, 9), f(21, 33)
    out.update(mm_a=a, mm_b=b, mm_c=c, mm_ab=R.matmul(a, b), mm_act=R.matmul_transpose_b(a, c))
    bias = f(9)
    out.update(lin_bias=bias, lin_out=R.linear(a.reshape(1, 17, 33), b, bias), addbias_out=R.add_bias(R.matmul(a, b), bias))
    table, pos = f(50, 24), f(12, 24)
    ids = rng.integers(0, 50, size=(3, 10)).astype(np.float32)
    emb = R.embedding_lookup(ids, table)
    out.update(emb_table=table, emb_pos=pos, emb_ids=ids, emb_out=emb, pos_out=R.add_positional_embedding(emb, pos),
               pos_at2_out=R.add_positional_embedding_at(emb, pos, 2))
    xi = f(2, 7, 64)
    w = [f(64, 64, scale=0.1) for _ in range(4)]
    out.update(attn_x=xi, attn_wq=w[0], attn_wk=w[1], attn_wv=w[2], attn_wo=w[3],
               attn_out=R.self_attention(xi, *w, 4))
    w1, b1, w2, b2 = f(64, 96, scale=0.1), f(96, scale=0.1), f(96, 64, scale=0.1), f(64, scale=0.1)
    out.update(ff_w1=w1, ff_b1=b1, ff_w2=w2, ff_b2=b2, ff_out=R.feed_forward(xi, w1, b1, w2, b2))
    q = np.concatenate([f(64, scale=50.0), np.array([0, np.inf, -np.inf, 448, 449, -500, 1e-9, -1e-9, 57344, 6e4, 1e30,
                                                    0.0625 + 1 / 256, 1.5, 2.5, 3.5], dtype=np.float32)])[None]
    out["q_x"] = q
    for dt in ("bf16", "fp16", "tf32", "fp8.e4m3", "fp8.e5m2"):
        out["q_" + dt.replace(".", "_")] = R.quantize(q, dt)
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **out)


def model_fixture():
    src = O.lm_source(seq=C1_SEQ, **C1)
    compiled = R.Compiled(src)
    ops = compiled.ops()
    assert ops == O.lm_ops(**C1)
    # (1) the `run` path without a checkpoint: seeded uniform(-0.1, 0.1) weights, seeded ids
    ids = compiled.synthetic_input(42, C1_BATCH)
    logits = compiled.executor_run(42, ids)
    model = R.Model(compiled, 42)
    names = model.param_names()
    first_rows = {n: model.param(i).reshape(-1)[:8] for i, n in enumerate(names)}
    np.savez_compressed(os.path.join(HERE, "c1_default.npz"), ids=ids, logits=logits,
                        names=np.array(names), **{"head_" + n: v for n, v in first_rows.items()})
    # (2) the checkpoint path: N(0, 0.02) weights written as BFCKPT1, loaded by the reference Model
    params = O.synth_params(ops, None, seed=7, sigma=0.02)
    ids2 = O.synth_token_ids(C1_BATCH, C1_SEQ, C1["vocab"], seed=11)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "c1.bfckpt")
        O.save_checkpoint(path, [(n, params[n]) for n in names])
        model.load_checkpoint(path)
        logits2 = model.forward(ids2)
        # and the reference's own writer, to pin the byte format
        back = os.path.join(tmp, "back.bfckpt")
        model.save_checkpoint(back)
        assert open(back, "rb").read() == open(path, "rb").read(), "BFCKPT1 writer mismatch"
    # simulated-precision forward of the CPU backend (storage bf16 / compute bf16)
    m_bf16 = R.Model(compiled, 42, {"storage": "bf16", "compute": "bf16"})
    for i, n in enumerate(names):
        m_bf16.set_param(i, params[n])
    np.savez_compressed(os.path.join(HERE, "c1_normal.npz"), ids=ids2, logits=logits2,
                        logits_cpu_bf16=m_bf16.forward(ids2), seed=np.array([7, 11]))


if __name__ == "__main__":
    ops_fixture()
    model_fixture()
    for name in sorted(os.listdir(HERE)):
        if name.endswith(".npz"):
            print(name, os.path.getsize(os.path.join(HERE, name)), "bytes")
