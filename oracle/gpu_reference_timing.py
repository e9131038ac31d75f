"""TEST INFRASTRUCTURE — times the reference's OWN CUDA backend (cuda::Model::forward with `compute bf16`: cuBLASLt
GEMMs, its fused attention kernel, its elementwise kernels; compiled unmodified into oracle/_ref/libbf_ref_cuda.so)
beside this repository's forward on the same GPU, the same model and the same token ids:

    python -m oracle.gpu_reference_timing [--batch 4] [--seq 2048] [--layers 16]

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
    args = ap.parse_args()

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


if __name__ == "__main__":
    main()
