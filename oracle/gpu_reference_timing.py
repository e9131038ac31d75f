"""TEST INFRASTRUCTURE — times the reference's OWN CUDA backend (cuda::Model::forward with `compute bf16`: cuBLASLt
GEMMs, its fused attention kernel, its elementwise kernels; compiled unmodified into oracle/_ref/libbf_ref_cuda.so)
beside this repository's forward on the same GPU, the same model and the same token ids:

    python -m oracle.gpu_reference_timing [--batch 4] [--seq 2048] [--layers 16]
    python -m oracle.gpu_reference_timing --decode [--batch 32] [--context 1920] [--steps 4]
    python -m oracle.gpu_reference_timing --gemm [--rows 65536] [--seconds 1.0]
    python -m oracle.gpu_reference_timing --attention-bwd [--batch 1] [--heads 2] [--seq 2048]

The first form also reports how far the two sets of logits are apart (largest difference over the largest logit, raw
top-1 agreement, agreement on the positions the reference decides by more than 2e-2 of the largest logit). `--gemm`
times the library call the reference's bf16Gemm makes (cublasLtMatmul with its settings, ops_tensorcore.cu:156-304)
beside this repository's tcgen05 GEMM on the five GEMM shapes of the 2B-class step, each for about a second of
back-to-back launches (so both run at the clocks the power cap allows), alternating, with the SM clock sampled.

The reference keeps the activations of every layer for its backward pass and an fp32 gradient beside every weight, so
it holds a slice of the headline batch (4 of the 32 sequences by default), not all of it. Both sides use their seeded
default initialisation (the same values). `--attention-bwd` times the reference's fusedAttentionBackward (fp32, CUDA
cores) beside this repository's tensor-core backward on the same bf16-valued operands and reports how far the gradients
are apart. Prints one JSON line."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--decode", action="store_true", help="time single-token generation steps after a prompt instead")
    ap.add_argument("--context", type=int, default=1920)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--gemm", action="store_true", help="cublasLtMatmul as the reference calls it against the tcgen05 GEMM")
    ap.add_argument("--rows", type=int, default=65536, help="--gemm: rows of A (tokens of a step)")
    ap.add_argument("--seconds", type=float, default=1.0, help="--gemm: length of each timed run")
    ap.add_argument("--attention-bwd", action="store_true", help="the reference's fusedAttentionBackward against the tcgen05 backward")
    ap.add_argument("--heads", type=int, default=2, help="--attention-bwd: heads of 128")
    args = ap.parse_args()
    if args.attention_bwd:
        return attention_backward(args)
    if args.decode:
        return decode(args)
    if args.gemm:
        return gemm_ab(args)

    import torch
    import blackforge_b200 as bfb
    from oracle import bf_oracle as O
    from oracle import ref_lib

    cfg = dict(vocab=32000, dim=2048, layers=args.layers, heads=16, hidden=5632, max_seq=args.seq)
    ids = O.synth_token_ids(args.batch, args.seq, cfg["vocab"], seed=7)
    policy = {"storage": "fp32", "compute": "bf16", "accumulate": "fp32"}

    ref = ref_lib.CudaModel(O.lm_source(seq=args.seq, **cfg), seed=42, precision=policy)
    ref_ms = ref.forward_timed(ids, warmup=1, iters=args.iters)
    ref_logits = ref.forward(ids)
    ref.close()

    ours = bfb.Model(O.lm_ops(**cfg), seed=42, precision={"storage": "bf16", "compute": "bf16"})
    d_ids = bfb.DeviceBuffer.from_numpy(np.ascontiguousarray(ids, dtype=np.float32))
    for _ in range(2):
        out, _ = ours.forward_device(d_ids.ptr, ids.shape, trusted=True)
        out.free()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iters):
        out, _ = ours.forward_device(d_ids.ptr, ids.shape, trusted=True)
        out.free()
    b.record()
    torch.cuda.synchronize()
    our_ms = a.elapsed_time(b) / args.iters
    tokens = args.batch * args.seq
    got = ours.forward_host(ids)
    scale = float(np.max(np.abs(ref_logits)))
    top2 = np.sort(ref_logits, axis=-1)[..., -2:]
    decided = (top2[..., 1] - top2[..., 0]) > 2e-2 * scale
    agree = np.argmax(got, axis=-1) == np.argmax(ref_logits, axis=-1)
    diff = {"max_abs_over_max": float(np.max(np.abs(got - ref_logits))) / scale, "top1_raw": float(agree.mean()),
            "decided_fraction": float(decided.mean()),
            "top1_decided": float(agree[decided].mean()) if decided.any() else None}
    print(json.dumps({"model": cfg, "batch": args.batch, "seq": args.seq,
                      "reference_cuda_ms": ref_ms, "reference_cuda_tokens_per_s": tokens / (ref_ms / 1e3),
                      "this_ms": our_ms, "this_tokens_per_s": tokens / (our_ms / 1e3), "ratio": ref_ms / our_ms,
                      "logits_vs_reference": diff}))


def attention_backward(args):
    import blackforge_b200 as bfb
    from oracle import bf_oracle as O
    from oracle import ref_lib

    batch = args.batch if args.batch != 4 else 1
    heads, seq, hd = args.heads, args.seq, 128
    dim = heads * hd
    rng = np.random.default_rng(5)
    q, k, v, g = (O.round_bf16(rng.standard_normal((batch, seq, dim)).astype(np.float32)) for _ in range(4))
    scale = float(hd ** -0.5)
    ref = ref_lib.cuda_fused_attention_backward(g, q, k, v, heads, scale, 0, iters=args.iters)
    lib = bfb.lib()
    dev = {n: bfb.upload(t, bfb.BF16) for n, t in (("g", g), ("q", q), ("k", k), ("v", v), ("o", O.round_bf16(ref["out"])))}
    d_m, d_l = bfb.upload(ref["m"], bfb.F32), bfb.upload(ref["l"], bfb.F32)
    grads = [bfb.DeviceBuffer(q.size * 4) for _ in range(3)]
    scratch = bfb.DeviceBuffer(batch * heads * seq * 8)
    status = bfb.DeviceBuffer.zeros(4)

    def run():
        bfb.check(lib.bfb_attention_bwd(dev["g"].ptr, dev["q"].ptr, dev["k"].ptr, dev["v"].ptr, dev["o"].ptr, d_m.ptr, d_l.ptr,
                                        grads[0].ptr, grads[1].ptr, grads[2].ptr, scratch.ptr, bfb.BF16, batch, seq, seq,
                                        heads, hd, dim, dim, dim, dim, scale, 0, 1, status.ptr, None))
    import torch
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.iters):
        run()
    e.record()
    torch.cuda.synchronize()
    ours_ms = s.elapsed_time(e) / args.iters
    flops = 10.0 * hd * batch * heads * seq * (seq + 1) / 2.0
    diffs = {}
    for name, buf in zip(("dq", "dk", "dv"), grads):
        got = bfb.download(buf, bfb.F32, q.shape)
        diffs[name] = float(np.max(np.abs(got - ref[name])) / np.max(np.abs(ref[name])))
    print(json.dumps({"what": "attention backward, causal, bf16-valued operands", "batch": batch, "heads": heads, "seq": seq,
                      "reference_ms": ref["ms"], "reference_tflops": flops / (ref["ms"] * 1e-3) / 1e12, "ours_ms": ours_ms,
                      "ours_tflops": flops / (ours_ms * 1e-3) / 1e12, "speedup": ref["ms"] / ours_ms,
                      "max_abs_diff_over_max_abs": diffs, "device_status": int(status.to_numpy(np.int32, (1,))[0])}))
    return 0


def gemm_ab(args):
    import subprocess
    import torch
    import blackforge_b200 as bfb
    from oracle import ref_lib

    lib = bfb.lib()
    m = args.rows
    # (name, n, k, C format of the step's launch)
    shapes = [("out-projection", 2048, 2048, "bf16"), ("QKV", 6144, 2048, "bf16"), ("feed-forward up", 5632, 2048, "bf16"),
              ("feed-forward down", 2048, 5632, "bf16"), ("logits", 32000, 2048, "f32")]

    def rand_bf16(count, scale):
        t = torch.randn(count, device="cuda", dtype=torch.float32) * scale
        buf = bfb.DeviceBuffer(count * 2)
        bfb.check(lib.bfb_cast(t.data_ptr(), bfb.F32, buf.ptr, bfb.BF16, count, 1.0, None, None))
        torch.cuda.synchronize()
        return buf

    # SM clock samples every 100 ms for the whole run, read by a thread; a timed run takes the median of its window
    import statistics
    import threading
    import time
    samples = []
    try:
        smi = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-lms", "100"],
                               stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)

        def reader():
            for line in smi.stdout:
                try:
                    samples.append((time.time(), float(line.strip())))
                except ValueError:
                    pass
        threading.Thread(target=reader, daemon=True).start()
    except OSError:
        smi = None

    def clocked(fn):
        t0 = time.time()
        ms = fn()
        t1 = time.time()
        time.sleep(0.12)
        inside = [v for (t, v) in samples if t0 + 0.2 <= t <= t1]
        return ms, (statistics.median(inside) if inside else None)

    status = bfb.DeviceBuffer.zeros(4)
    rows = []
    for name, n, k, cfmt in shapes:
        a = rand_bf16(m * k, 1.0)
        w_nk = rand_bf16(n * k, 0.02)      # this repository's layout: W^T [n, k]
        w_kn = rand_bf16(k * n, 0.02)      # the reference's layout: W [k, n]
        c = bfb.DeviceBuffer(m * n * 4)         # large enough for either result format
        cd = bfb.BF16 if cfmt == "bf16" else bfb.F32
        flops = 2.0 * m * n * k

        def ours(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                bfb.check(lib.bfb_gemm(a.ptr, w_nk.ptr, c.ptr, m, n, k, bfb.BF16, bfb.B_NK, cd, bfb.EPI["none"], None, None,
                                       1.0, None, 0, status.ptr, None))
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / iters

        def theirs(iters, c_bf16):
            return ref_lib.cuda_lt_gemm_timed(a.ptr, w_kn.ptr, c.ptr, m, n, k, c_bf16, 0, iters)

        est = max(ours(3), 1e-3)
        iters = max(3, int(args.seconds * 1e3 / est))
        entry = {"gemm": name, "m": m, "n": n, "k": k, "c": cfmt, "iters": iters}
        # alternate so that neither side always runs on the warmer chip; the clock is read right after each run
        for rep in range(2):
            t, mhz = clocked(lambda: ours(iters))
            entry.setdefault("this_tflops", []).append(flops / (t / 1e3) / 1e12)
            entry.setdefault("this_sm_mhz", []).append(mhz)
            t, mhz = clocked(lambda: theirs(iters, cfmt == "bf16"))
            entry.setdefault("cublaslt_tflops", []).append(flops / (t / 1e3) / 1e12)
            entry.setdefault("cublaslt_sm_mhz", []).append(mhz)
        if cfmt == "bf16":
            t, mhz = clocked(lambda: theirs(iters, False))
            entry["cublaslt_f32_result_tflops"] = flops / (t / 1e3) / 1e12   # the reference's own result format
        entry["ratio"] = max(entry["this_tflops"]) / max(entry["cublaslt_tflops"])
        rows.append(entry)
        for buf in (a, w_nk, w_kn, c):
            buf.free()
        bfb.check(lib.bfb_pool_trim())
    if smi is not None:
        smi.terminate()
    print(json.dumps({"rows_of_a": m, "seconds_per_run": args.seconds, "gemms": rows,
                      "note": "cublasLtMatmul with the reference's settings (row-major bf16 A [m,k] and B [k,n], fp32 "
                              "compute, heuristic top-1, 4 MiB workspace); this repository's kernel reads W^T [n,k]"}))


def decode(args):
    import torch
    import blackforge_b200 as bfb
    from oracle import bf_oracle as O
    from oracle import ref_lib

    batch = args.batch if args.batch != 4 else 32
    max_seq = args.context + args.steps + 2
    cfg = dict(vocab=32000, dim=2048, layers=args.layers, heads=16, hidden=5632, max_seq=max_seq)
    ids = O.synth_token_ids(batch, args.context + args.steps + 1, cfg["vocab"], seed=7)
    prompt, steps = ids[:, :args.context], ids[:, args.context:args.context + args.steps]
    policy = {"storage": "fp32", "compute": "bf16", "accumulate": "fp32"}

    ours = bfb.Model(O.lm_ops(**cfg), seed=42, precision={"storage": "bf16", "compute": "bf16"})
    d_prompt = bfb.DeviceBuffer.from_numpy(np.ascontiguousarray(prompt, dtype=np.float32))
    d_steps = [bfb.DeviceBuffer.from_numpy(np.ascontiguousarray(ids[:, args.context + i:args.context + i + 1], dtype=np.float32))
               for i in range(args.steps + 1)]
    ours.reset_generation()
    out, _ = ours.forward_incremental_device(d_prompt.ptr, prompt.shape, trusted=True)
    out.free()
    out, _ = ours.forward_incremental_device(d_steps[0].ptr, (batch, 1), trusted=True)   # warm-up step
    out.free()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(args.steps):
        out, _ = ours.forward_incremental_device(d_steps[1 + i].ptr, (batch, 1), trusted=True)
        out.free()
    b.record()
    torch.cuda.synchronize()
    our_ms = a.elapsed_time(b) / args.steps
    # this side first, and its memory handed back: the reference's device pool never returns memory, and its caches
    # grow by re-allocation (a new size every step), so it needs most of the device for a handful of steps
    ours.close()
    for buf in [d_prompt] + d_steps:
        buf.free()
    bfb.check(bfb.lib().bfb_pool_trim())
    torch.cuda.empty_cache()
    ref = ref_lib.CudaModel(O.lm_source(seq=max_seq, **cfg), seed=42, precision=policy)
    ref_ms = ref.generation_timed(prompt, steps)
    ref.close()
    print(json.dumps({"model": cfg, "batch": batch, "context": args.context, "steps": args.steps,
                      "reference_cuda_ms_per_step": ref_ms, "reference_cuda_tokens_per_s": batch / (ref_ms / 1e3),
                      "this_ms_per_step": our_ms, "this_tokens_per_s": batch / (our_ms / 1e3), "ratio": ref_ms / our_ms}))


if __name__ == "__main__":
    main()
