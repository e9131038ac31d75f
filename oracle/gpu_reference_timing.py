"""TEST INFRASTRUCTURE — times the reference's OWN CUDA backend (cuda::Model::forward with `compute bf16`: cuBLASLt
GEMMs, its fused attention kernel, its elementwise kernels; compiled unmodified into oracle/_ref/libbf_ref_cuda.so)
beside this repository's forward on the same GPU, the same model and the same token ids:

    python -m oracle.gpu_reference_timing [--batch 4] [--seq 2048] [--layers 16]
    python -m oracle.gpu_reference_timing --decode [--batch 32] [--context 1920] [--steps 4]

The reference keeps the activations of every layer for its backward pass and an fp32 gradient beside every weight, so
it holds a slice of the headline batch (4 of the 32 sequences by default), not all of it. Both sides use their seeded
default initialisation (the same values). Prints one JSON line."""
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
    args = ap.parse_args()
    if args.decode:
        return decode(args)

    import torch
    import blackforge_b200 as bfb
    from oracle import bf_oracle as O
    from oracle import ref_lib

    cfg = dict(vocab=32000, dim=2048, layers=args.layers, heads=16, hidden=5632, max_seq=args.seq)
    ids = O.synth_token_ids(args.batch, args.seq, cfg["vocab"], seed=7)
    policy = {"storage": "fp32", "compute": "bf16", "accumulate": "fp32"}

    ref = ref_lib.CudaModel(O.lm_source(seq=args.seq, **cfg), seed=42, precision=policy)
    ref_ms = ref.forward_timed(ids, warmup=1, iters=args.iters)
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
    print(json.dumps({"model": cfg, "batch": args.batch, "seq": args.seq,
                      "reference_cuda_ms": ref_ms, "reference_cuda_tokens_per_s": tokens / (ref_ms / 1e3),
                      "this_ms": our_ms, "this_tokens_per_s": tokens / (our_ms / 1e3), "ratio": ref_ms / our_ms}))


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
