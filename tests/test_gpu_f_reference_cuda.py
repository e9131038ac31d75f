"""This repository's kernels against the reference's OWN CUDA backend on the same inputs: blackforge::backend::cuda::Model
with `compute bf16` (its cuBLASLt path, src/backend/cuda/ops_tensorcore.cu) and fusedAttentionForward
(src/backend/cuda/fused_attention.cu), compiled unmodified into oracle/_ref/libbf_ref_cuda.so. Skipped where that
library was not built (it needs the reference's sources at build time, not at run time)."""
import numpy as np
import pytest

from oracle import bf_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refcuda():
    from oracle import ref_lib
    if not ref_lib.cuda_available():
        pytest.skip("oracle/_ref/libbf_ref_cuda.so not built")
    return ref_lib


def _reference_logits(refcuda, cfg, seq, params, ids, precision):
    model = refcuda.CudaModel(O.lm_source(seq=seq, **cfg), seed=1, precision=precision)
    names = model.param_names()
    assert sorted(names) == sorted(params)
    for i, n in enumerate(names):
        model.set_param(i, params[n])
    out = model.forward(ids)
    model.close()
    return out


@pytest.mark.parametrize("cfg,batch,seq,sigma", [
    (dict(vocab=1024, dim=512, layers=2, heads=4, hidden=1024, max_seq=256), 2, 256, 0.05),
    # the 2B-class configuration's layer shapes (d 2048, 16 heads of 128, ffn 5632, vocabulary 32000), two layers, one
    # sequence of 512: a slice of the headline workload the reference's device path can hold
    (dict(vocab=32000, dim=2048, layers=2, heads=16, hidden=5632, max_seq=512), 1, 512, 0.02),
])
def test_bf16_model_against_the_reference_cublaslt_path(gpu, refcuda, cfg, batch, seq, sigma):
    """The stated bf16 criterion: within 2e-2 of the reference's cuBLASLt path, and the same top-1 token on at least
    99.5 % of the positions where the reference's own decision is not a near tie."""
    ops = O.lm_ops(**cfg)
    params = O.synth_params(ops, None, seed=31, sigma=sigma, bias_sigma=sigma)
    ids = O.synth_token_ids(batch, seq, cfg["vocab"], seed=32)
    want = _reference_logits(refcuda, cfg, seq, params, ids, {"storage": "fp32", "compute": "bf16", "accumulate": "fp32"})
    ours = gpu.Model(ops, precision={"storage": "fp32", "compute": "bf16"}, random_init=False)
    ours.set_params(params)
    got = ours.forward_host(ids)
    assert got.shape == want.shape
    scale = float(np.max(np.abs(want)))
    print("bf16 vs reference cuBLASLt path: max abs diff / max abs =", float(np.max(np.abs(got - want))) / scale)
    assert float(np.max(np.abs(got - want))) <= 2e-2 * scale
    top2 = np.sort(want, axis=-1)[..., -2:]
    decided = (top2[..., 1] - top2[..., 0]) > 2e-2 * scale
    agree = np.argmax(got, axis=-1) == np.argmax(want, axis=-1)
    print("decided positions", float(decided.mean()), "top-1 agreement on them", float(agree[decided].mean()))
    assert decided.mean() > 0.2 and agree[decided].mean() >= 0.995


def logit_differences(got, want):
    """The figures the bf16 criterion is stated in, all of them: the largest difference relative to the largest logit,
    RAW top-1 agreement over every position, and agreement on the positions the reference decides by more than the
    2e-2 bar (with the share of positions that is)."""
    scale = float(np.max(np.abs(want)))
    top2 = np.sort(want, axis=-1)[..., -2:]
    decided = (top2[..., 1] - top2[..., 0]) > 2e-2 * scale
    agree = np.argmax(got, axis=-1) == np.argmax(want, axis=-1)
    return {"max_abs_over_max": float(np.max(np.abs(got - want))) / scale,
            "rel_l2": float(np.sqrt(np.sum((got - want) ** 2) / np.sum(want ** 2))),
            "top1_raw": float(agree.mean()), "decided_fraction": float(decided.mean()),
            "top1_decided": float(agree[decided].mean()) if decided.any() else float("nan")}


def _set_all(model, params, names):
    for i, n in enumerate(names):
        model.set_param(i, params[n])


def test_benchmarked_route_at_full_depth_against_the_reference_cublaslt_path(gpu, refcuda):
    """The route the benchmark times, {storage bf16, compute bf16} (bf16 residual stream, rmsnorm folded into the GEMM
    epilogues), on the 2B-class model at its full depth: 16 layers, d 2048, 16 heads of 128, ffn 5632, vocabulary
    32000, weights N(0, 0.02) as the benchmark configuration states, two whole sequences of 2048 tokens, against the
    reference's own device path with `compute bf16` (its cuBLASLt GEMMs on fp32 activations, model.cu:252-306,
    ops_tensorcore.cu:293-327). The rounding of the residual stream grows with depth, so this is the case that
    decides whether the timed route meets the 2e-2 bar; the fp32-stream route is measured beside it. How much bf16
    rounding moves THIS model at all is measured too: the reference's bf16 path against the reference's own fp32
    path (cublasSgemm). All figures are printed."""
    cfg = dict(vocab=32000, dim=2048, layers=16, heads=16, hidden=5632, max_seq=2048)
    batch, seq = 2, 2048
    ops = O.lm_ops(**cfg)
    params = O.synth_params(ops, None, seed=41, sigma=0.02, bias_sigma=0.02)
    ids = O.synth_token_ids(batch, seq, cfg["vocab"], seed=7)
    source = O.lm_source(seq=seq, **cfg)

    def reference(precision):
        ref = refcuda.CudaModel(source, seed=1, precision=precision)
        _set_all(ref, params, ref.param_names())
        out = ref.forward(ids)
        ref.close()
        return out

    want = reference({"storage": "fp32", "compute": "bf16", "accumulate": "fp32"})
    results = {"reference fp32 path vs its bf16 path": logit_differences(reference(None), want)}
    for storage in ("bf16", "fp32"):
        ours = gpu.Model(ops, precision={"storage": storage, "compute": "bf16"}, random_init=False)
        ours.set_params(params)
        got = ours.forward_host(ids)
        ours.close()
        gpu.check(gpu.lib().bfb_pool_trim())
        assert got.shape == want.shape == (batch, seq, cfg["vocab"])
        results[storage] = logit_differences(got, want)
    for name, r in results.items():
        print(f"16 layers, 2 x 2048 tokens, N(0, 0.02) weights, {name}:", r)
    for storage in ("bf16", "fp32"):
        r = results[storage]
        assert r["max_abs_over_max"] <= 2e-2, (storage, r)
        assert r["top1_decided"] >= 0.995, (storage, r)
    # raw agreement: random-weight logits have many near ties (the two best logits closer than the bf16 noise), which
    # no bf16 implementation decides the same way; the figure is recorded, and must not fall far below the bar
    assert results["bf16"]["top1_raw"] >= 0.97, results["bf16"]


def test_seeded_default_weights_at_full_depth_are_ill_conditioned_for_everyone(gpu, refcuda):
    """The same comparison on the reference's seeded default weights (uniform(-0.1, 0.1), seed 42: the values both
    sides draw when no checkpoint is given). At d 2048 every projection then multiplies the norm by about 2.6 and the
    attention scores have a spread of several units, so after 16 layers bf16 rounding anywhere moves the logits by a
    tenth of their range: the reference's own bf16 path is that far from the reference's own fp32 path. No bar can be
    asserted against such a target beyond "no further from the reference's bf16 path than its own fp32 path is";
    the figures are printed."""
    cfg = dict(vocab=32000, dim=2048, layers=16, heads=16, hidden=5632, max_seq=2048)
    batch, seq = 2, 2048
    ids = O.synth_token_ids(batch, seq, cfg["vocab"], seed=7)
    source = O.lm_source(seq=seq, **cfg)

    def reference(precision):
        ref = refcuda.CudaModel(source, seed=42, precision=precision)
        out = ref.forward(ids)
        ref.close()
        return out

    want = reference({"storage": "fp32", "compute": "bf16", "accumulate": "fp32"})
    own = logit_differences(reference(None), want)
    print("16 layers, default uniform(-0.1, 0.1) weights, reference fp32 path vs its bf16 path:", own)
    for storage in ("bf16", "fp32"):
        ours = gpu.Model(O.lm_ops(**cfg), seed=42, precision={"storage": storage, "compute": "bf16"})
        got = ours.forward_host(ids)
        ours.close()
        gpu.check(gpu.lib().bfb_pool_trim())
        r = logit_differences(got, want)
        print(f"16 layers, default uniform(-0.1, 0.1) weights, storage {storage} vs reference cuBLASLt path:", r)
        assert r["rel_l2"] <= 2.0 * own["rel_l2"] + 2e-2, (storage, r, own)


def test_fp32_model_against_the_reference_device_path(gpu, refcuda):
    cfg = dict(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32)
    ops = O.lm_ops(**cfg)
    params = O.synth_params(ops, None, seed=33, sigma=0.05, bias_sigma=0.05)
    ids = O.synth_token_ids(4, 32, cfg["vocab"], seed=34)
    want = _reference_logits(refcuda, cfg, 32, params, ids, None)
    ours = gpu.Model(ops, random_init=False)
    ours.set_params(params)
    err = float(np.max(np.abs(ours.forward_host(ids) - want)))
    print("fp32 vs reference device path: max abs diff", err)
    assert err <= 1e-3


@pytest.mark.parametrize("old_len", [0, 96])
def test_attention_against_the_reference_fused_kernel(gpu, refcuda, old_len):
    """tcgen05 flash attention (bf16) against fusedAttentionForward on the same bf16-valued inputs in fp32."""
    rng = np.random.default_rng(41 + old_len)
    batch, heads, new_len = 2, 4, 256
    total, dim = old_len + new_len, heads * 128
    q = O.round_bf16(rng.standard_normal((batch, new_len, dim)).astype(np.float32))
    k = O.round_bf16(rng.standard_normal((batch, total, dim)).astype(np.float32))
    v = O.round_bf16(rng.standard_normal((batch, total, dim)).astype(np.float32))
    scale = float(128 ** -0.5)
    want = refcuda.cuda_fused_attention(q, k, v, heads, scale, old_len)
    d_q, d_k, d_v = (gpu.upload(t, gpu.BF16) for t in (q, k, v))
    d_o = gpu.DeviceBuffer(batch * new_len * dim * 2)
    d_status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_attention_fwd(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, None, None, gpu.BF16, batch, new_len, total,
                                          heads, 128, dim, dim, dim, dim, scale, old_len, 1, d_status.ptr, None))
    got = gpu.download(d_o, gpu.BF16, (batch, new_len, dim))
    assert int(d_status.to_numpy(np.int32, (1,))[0]) == 0
    print("attention vs reference fused kernel: max abs diff", float(np.max(np.abs(got - want))))
    assert float(np.max(np.abs(got - want))) <= 1.2e-2


@pytest.mark.parametrize("precision", [None, {"storage": "fp32", "compute": "bf16", "accumulate": "fp32"}])
def test_generation_steps_against_the_reference_key_value_cache(gpu, refcuda, precision):
    """Model::forwardIncremental here (in-place caches, one-query attention, few-rows GEMMs on the bf16 route) against
    the reference's own cuda::Model::forwardIncremental: a prompt, then single-token steps, same weights and ids."""
    cfg = dict(vocab=512, dim=256, layers=2, heads=2, hidden=512, max_seq=96)
    ops = O.lm_ops(**cfg)
    params = O.synth_params(ops, None, seed=51, sigma=0.05, bias_sigma=0.05)
    ids = O.synth_token_ids(3, 70, cfg["vocab"], seed=52)
    theirs = refcuda.CudaModel(O.lm_source(seq=96, **cfg), seed=1, precision=precision)
    for i, n in enumerate(theirs.param_names()):
        theirs.set_param(i, params[n])
    ours = gpu.Model(ops, precision=None if precision is None else {"storage": "fp32", "compute": "bf16"}, random_init=False)
    ours.set_params(params)
    theirs.reset_generation()
    ours.reset_generation()
    bar = 1e-3 if precision is None else 2e-2
    worst = 0.0
    for lo, hi in ((0, 64), (64, 65), (65, 66), (66, 70)):
        want = theirs.forward_incremental(ids[:, lo:hi])
        got = ours.forward_incremental(ids[:, lo:hi])
        assert got.shape == want.shape
        worst = max(worst, float(np.max(np.abs(got - want))) / float(np.max(np.abs(want))))
    print("generation vs reference key/value cache: worst max abs diff / max abs =", worst)
    assert worst <= bar
    theirs.close()


def test_attention_configuration_2_in_full_against_the_reference_kernel(gpu, refcuda):
    """Configuration 2 at its full size (batch 16, 16 heads of 128, sequence 2048, causal): every output element of
    the tcgen05 kernel against the reference's fused kernel on the same bf16-valued inputs, and both device times."""
    rng = np.random.default_rng(2)
    batch, heads, seq = 16, 16, 2048
    dim = heads * 128
    q, k, v = (O.round_bf16(rng.standard_normal((batch, seq, dim), dtype=np.float32)) for _ in range(3))
    scale = float(128 ** -0.5)
    want, ref_ms = refcuda.cuda_fused_attention_timed(q, k, v, heads, scale, 0, iters=2)
    d_q, d_k, d_v = (gpu.upload(t, gpu.BF16) for t in (q, k, v))
    d_o = gpu.DeviceBuffer(batch * seq * dim * 2)
    d_status = gpu.DeviceBuffer.zeros(4)

    def run():
        gpu.check(gpu.lib().bfb_attention_fwd(d_q.ptr, d_k.ptr, d_v.ptr, d_o.ptr, None, None, gpu.BF16, batch, seq, seq, heads,
                                              128, dim, dim, dim, dim, scale, 0, 1, d_status.ptr, None))
    import torch
    run()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        run()
    b.record()
    torch.cuda.synchronize()
    our_ms = a.elapsed_time(b) / 5
    got = gpu.download(d_o, gpu.BF16, (batch, seq, dim))
    assert int(d_status.to_numpy(np.int32, (1,))[0]) == 0
    err = float(np.max(np.abs(got - want)))
    flops = 4.0 * 128 * batch * heads * seq * (seq + 1) / 2.0
    print(f"configuration 2 vs reference fused kernel: max abs diff {err:.3e}; reference {ref_ms:.2f} ms "
          f"({flops / ref_ms / 1e9:.1f} TFLOP/s causal), this kernel {our_ms:.3f} ms ({flops / our_ms / 1e9:.1f} TFLOP/s)")
    assert err <= 1.2e-2
