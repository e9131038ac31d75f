"""Writes tests/golden/attention_backward.npz: inputs and the outputs of the reference's own fusedAttentionForward +
fusedAttentionBackward (src/backend/cuda/fused_attention.cu:305-380, compiled unmodified into
oracle/_ref/libbf_ref_cuda.so) for two seeded cases. Needs a CUDA device; run from the repository root:

    python tests/golden/make_attention_backward_golden.py [--out PATH]

Case "small": fp32 values, 2 x 3 heads of 16, 11 new rows after 6 cached ones. Case "hd128": bf16-valued inputs,
2 heads of 128, 200 new rows after 72 cached ones (the tensor-core route's shape class)."""
import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import bf_oracle as O  # noqa: E402
from oracle import ref_lib  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "attention_backward.npz"))
    args = ap.parse_args()
    rng = np.random.default_rng(20240611)
    blob = {}
    for tag, (B, H, D, old, new, bf16) in {"small": (2, 3, 16, 6, 11, False), "hd128": (1, 2, 128, 72, 200, True)}.items():
        r = O.round_bf16 if bf16 else (lambda x: x)
        q = r(rng.standard_normal((B, new, H * D)).astype(np.float32))
        k = r(rng.standard_normal((B, old + new, H * D)).astype(np.float32))
        v = r(rng.standard_normal((B, old + new, H * D)).astype(np.float32))
        g = r(rng.standard_normal((B, new, H * D)).astype(np.float32))
        res = ref_lib.cuda_fused_attention_backward(g, q, k, v, H, float(1.0 / np.sqrt(np.float32(D))), old)
        blob.update({f"{tag}_d_out": g, f"{tag}_q": q, f"{tag}_k": k, f"{tag}_v": v, f"{tag}_heads": np.int64(H),
                     f"{tag}_old_len": np.int64(old)})
        blob.update({f"{tag}_{n}": res[n] for n in ("out", "m", "l", "dq", "dk", "dv")})
    np.savez_compressed(args.out, **blob)
    print("wrote", args.out, {n: a.shape for n, a in blob.items()})


if __name__ == "__main__":
    main()
