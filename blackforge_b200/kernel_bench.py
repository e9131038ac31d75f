"""Times ONE kernel of the library in isolation through the C ABI (CUDA events on the launching stream,
L2 flushed between iterations) and prints one JSON line. This is what the ncu captures under profiles/
run, on small cases.

    python -m blackforge_b200.kernel_bench gemm --m 65536 --n 2048 --k 2048 [--dtype bf16|fp8] [--epilogue none]
    python -m blackforge_b200.kernel_bench attention --batch 16 --heads 16 --seq 2048
    python -m blackforge_b200.kernel_bench attention-bwd --batch 8 --heads 16 --seq 2048
    python -m blackforge_b200.kernel_bench matmul-bwd --m 65536 --k 2048 --n 5632
    python -m blackforge_b200.kernel_bench rmsnorm --rows 65536 --dim 2048
    python -m blackforge_b200.kernel_bench embed --batch 32 --seq 2048 --vocab 32000 --dim 2048

and the checkpoint loader (host I/O + uploads, wall clock; the file is written first, so it comes from the page cache):

    python -m blackforge_b200.kernel_bench checkpoint --layers 16 [--dim 2048 --hidden 5632 --vocab 32000] [--path FILE]
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attention", "attention-bwd", "matmul-bwd", "rmsnorm", "embed", "checkpoint"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=5632)
    ap.add_argument("--chunk-mib", type=int, default=0, help="checkpoint: staging buffer size (0: the loader's default)")
    ap.add_argument("--path", default="", help="checkpoint: where to write the file (default: a temporary directory)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--cdtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--epilogue", default="none")
    ap.add_argument("--layout", default="nk", choices=["nk", "kn"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--stream-dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--decode-context", type=int, default=0,
                    help="attention: one new query per sequence against this many cached keys (a generation step)")
    ap.add_argument("--dynamic-tiles", action="store_true",
                    help="gemm: tiles drawn from a device counter (the mode for GEMMs that share the SMs)")
    ap.add_argument("--reserved-sms", type=int, default=0, help="size the persistent grids for this many fewer SMs")
    args = ap.parse_args()

    import torch
    import blackforge_b200 as bfb

    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a CUDA device")
    lib = bfb.lib()
    if args.kernel == "checkpoint":
        return checkpoint_io(args, bfb)
    if args.dynamic_tiles or args.reserved_sms:
        bfb.set_shared_sm_mode(args.dynamic_tiles, args.reserved_sms)
    rng = np.random.default_rng(0)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def rand_dev(count, dtype, scale=1.0):
        """Random device buffer in `dtype` without a host round trip of the full size in fp32."""
        t = torch.randn(count, device="cuda", dtype=torch.float32) * scale
        buf = bfb.DeviceBuffer(count * bfb.ELEM_BYTES[dtype])
        bfb.check(lib.bfb_cast(t.data_ptr(), bfb.F32, buf.ptr, dtype, count, 1.0, None, None))
        torch.cuda.synchronize()
        return buf

    status = bfb.DeviceBuffer.zeros(4)
    if args.kernel == "gemm":
        ab = bfb.BF16 if args.dtype == "bf16" else bfb.FP8_E4M3
        cd = bfb.BF16 if args.cdtype == "bf16" else bfb.F32
        a = rand_dev(args.m * args.k, ab)
        b = rand_dev(args.n * args.k, ab, 0.05)
        c = bfb.DeviceBuffer(args.m * args.n * bfb.ELEM_BYTES[cd])
        bias = rand_dev(args.n, bfb.F32)
        res = bfb.DeviceBuffer.zeros(args.m * args.n * bfb.ELEM_BYTES[cd])
        layout = bfb.B_NK if args.layout == "nk" else bfb.B_KN
        epi = bfb.EPI[args.epilogue]

        def run():
            bfb.check(lib.bfb_gemm(a.ptr, b.ptr, c.ptr, args.m, args.n, args.k, ab, layout, cd, epi, bias.ptr, res.ptr,
                                   1.0, None, 0, status.ptr, None))
        work, unit = 2.0 * args.m * args.n * args.k, "TFLOP/s"
        desc = {"m": args.m, "n": args.n, "k": args.k, "operands": args.dtype, "c": args.cdtype, "epilogue": args.epilogue,
                "b_layout": args.layout}
    elif args.kernel == "attention" and args.decode_context > 0:
        dim, ctx = args.heads * 128, args.decode_context
        q = rand_dev(args.batch * dim, bfb.BF16)
        k, v = (rand_dev(args.batch * ctx * dim, bfb.BF16) for _ in range(2))
        out = bfb.DeviceBuffer(args.batch * dim * 2)

        def run():
            bfb.check(lib.bfb_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, None, None, bfb.BF16, args.batch, 1, ctx,
                                            args.heads, 128, dim, dim, dim, dim, float(128 ** -0.5), ctx - 1, 1,
                                            status.ptr, None))
        work, unit = float(2 * args.batch * ctx * dim * 2), "GB/s"
        desc = {"batch": args.batch, "heads": args.heads, "context": ctx, "head_dim": 128, "bytes": "keys + values, bf16"}
    elif args.kernel == "attention":
        dim = args.heads * 128
        q, k, v = (rand_dev(args.batch * args.seq * dim, bfb.BF16) for _ in range(3))
        out = bfb.DeviceBuffer(args.batch * args.seq * dim * 2)

        def run():
            bfb.check(lib.bfb_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, None, None, bfb.BF16, args.batch, args.seq,
                                            args.seq, args.heads, 128, dim, dim, dim, dim, float(128 ** -0.5), 0, 1,
                                            status.ptr, None))
        work, unit = 4.0 * 128 * args.batch * args.heads * args.seq * (args.seq + 1) / 2.0, "TFLOP/s"
        desc = {"batch": args.batch, "heads": args.heads, "seq": args.seq, "head_dim": 128, "flops": "causal"}
    elif args.kernel == "attention-bwd":
        # the forward first (its output and row statistics are the backward's operands), then the backward alone is timed:
        # the statistics kernel, the zero fill of the three gradients and the tensor-core kernel
        dim = args.heads * 128
        q, k, v, g = (rand_dev(args.batch * args.seq * dim, bfb.BF16) for _ in range(4))
        out = bfb.DeviceBuffer(args.batch * args.seq * dim * 2)
        rows = args.batch * args.heads * args.seq
        m_, l_, scratch = bfb.DeviceBuffer(rows * 4), bfb.DeviceBuffer(rows * 4), bfb.DeviceBuffer(rows * 8)
        dq, dk, dv = (bfb.DeviceBuffer(args.batch * args.seq * dim * 4) for _ in range(3))
        bfb.check(lib.bfb_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, m_.ptr, l_.ptr, bfb.BF16, args.batch, args.seq, args.seq,
                                        args.heads, 128, dim, dim, dim, dim, float(128 ** -0.5), 0, 1, status.ptr, None))

        def run():
            bfb.check(lib.bfb_attention_bwd(g.ptr, q.ptr, k.ptr, v.ptr, out.ptr, m_.ptr, l_.ptr, dq.ptr, dk.ptr, dv.ptr,
                                            scratch.ptr, bfb.BF16, args.batch, args.seq, args.seq, args.heads, 128, dim, dim,
                                            dim, dim, float(128 ** -0.5), 0, 1, status.ptr, None))
        # five products of 2 * 128 flops per visible (query, key) pair
        work, unit = 10.0 * 128 * args.batch * args.heads * args.seq * (args.seq + 1) / 2.0, "TFLOP/s"
        desc = {"batch": args.batch, "heads": args.heads, "seq": args.seq, "head_dim": 128, "flops": "causal, 5 products"}
    elif args.kernel == "matmul-bwd":
        # both gradients of C = A B from fp32 tensors, as the reference's matmulBf16Backward takes them: three casts to
        # bf16 (two of them transposing) and two tensor-core GEMMs
        a = rand_dev(args.m * args.k, bfb.F32)
        b = rand_dev(args.k * args.n, bfb.F32, 0.05)
        g = rand_dev(args.m * args.n, bfb.F32)
        d_a, d_b = bfb.DeviceBuffer(args.m * args.k * 4), bfb.DeviceBuffer(args.k * args.n * 4)

        def run():
            bfb.check(lib.bfb_matmul_bf16_backward(a.ptr, b.ptr, g.ptr, d_a.ptr, d_b.ptr, args.m, args.k, args.n, None))
        work, unit = 4.0 * args.m * args.k * args.n, "TFLOP/s"
        desc = {"m": args.m, "k": args.k, "n": args.n, "operands": "fp32 in, bf16 products, fp32 out", "flops": "dA and dB"}
    elif args.kernel == "rmsnorm":
        sd = bfb.BF16 if args.stream_dtype == "bf16" else bfb.F32
        x = rand_dev(args.rows * args.dim, sd)
        out = bfb.DeviceBuffer(args.rows * args.dim * 2)

        def run():
            bfb.check(lib.bfb_rmsnorm(x.ptr, sd, out.ptr, bfb.BF16, args.rows, args.dim, 1e-6, None))
        work, unit = float(args.rows * args.dim * (bfb.ELEM_BYTES[sd] + 2)), "GB/s"
        desc = {"rows": args.rows, "dim": args.dim, "in": args.stream_dtype, "out": "bf16"}
    else:
        sd = bfb.BF16 if args.stream_dtype == "bf16" else bfb.F32
        table = rand_dev(args.vocab * args.dim, bfb.F32)
        pos = rand_dev(args.seq * args.dim, bfb.F32)
        ids = bfb.DeviceBuffer.from_numpy(rng.integers(0, args.vocab, size=(args.batch, args.seq)).astype(np.float32))
        out = bfb.DeviceBuffer(args.batch * args.seq * args.dim * bfb.ELEM_BYTES[sd])

        def run():
            bfb.check(lib.bfb_embed_pos(ids.ptr, table.ptr, pos.ptr, out.ptr, sd, args.batch, args.seq, args.vocab,
                                        args.dim, args.seq, 0, None, None))
        work, unit = float(args.batch * args.seq * args.dim * (8 + bfb.ELEM_BYTES[sd])), "GB/s"
        desc = {"batch": args.batch, "seq": args.seq, "vocab": args.vocab, "dim": args.dim, "out": args.stream_dtype}

    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.iters):
        if flush is not None:
            flush.zero_()            # 256 MiB write: evicts the 126 MB L2
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    st = int(status.to_numpy(np.int32, (1,))[0])
    ms = float(np.median(times))
    rate = work / (ms / 1e3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"kernel": args.kernel, "case": desc, "ms_median": ms, "ms_min": float(min(times)), "rate": rate,
                      "unit": unit, "iters": args.iters, "l2_flushed": flush is not None, "device_status": st}))
    return 0 if st == 0 else 1


def checkpoint_io(args, bfb):
    """Writes a BFCKPT1 file of a decoder of the given shape (weights drawn on the device), then times the streaming
    loader into a fresh model, and the reference's way of loading (each tensor whole into pageable host memory, one
    synchronous upload per tensor) beside it."""
    import tempfile
    import time

    ops, vid = [], 0
    for kind, kw in ([("embedding", dict(vocab=args.vocab, emb_dim=args.dim)), ("positional_embedding", dict(max_seq=args.seq))]
                     + [("attention", dict(heads=args.dim // 128)), ("feedforward", dict(hidden=args.hidden))] * args.layers
                     + [("linear", dict(linear_out=args.vocab))]):
        ops.append(dict(kind=kind, input=vid, output=vid + 1, **kw))
        vid += 1
    src = bfb.Model(ops, random_init=False)
    for i, _ in enumerate(src.param_names()):
        src.fill_param_normal(i, 1000 + i, 0.02)
    with tempfile.TemporaryDirectory() as tmp:
        path = args.path or f"{tmp}/weights.bfckpt"
        t0 = time.perf_counter()
        src.save_checkpoint(path)
        save_s = time.perf_counter() - t0
        src.close()
        index = bfb.checkpoint_index(path)
        runs = []
        for _ in range(max(1, args.iters // 5)):
            dst = bfb.Model(ops, random_init=False)
            runs.append(dst.load_checkpoint_streaming(path, args.chunk_mib << 20))
            dst.close()
        best = min(runs, key=lambda r: r["seconds"])
        # with the cache of converted weights beside the file: first load writes it, later ones read it
        cached = {}
        if args.dtype in ("bf16", "fp8"):
            prec = {"storage": "bf16", "compute": "bf16" if args.dtype == "bf16" else "fp8.e4m3"}
            for label in ("miss", "hit", "hit_again"):
                dst = bfb.Model(ops, precision=prec, random_init=False)
                r = dst.load_checkpoint_cached(path, args.chunk_mib << 20)
                dst.close()
                cached[label] = {"seconds": r["seconds"], "read_gb": r["read_bytes"] / 1e9, "cache_hit": r["cache_hit"]}
        # the reference's order of work: read a tensor whole, upload it synchronously, next tensor
        dst = bfb.Model(ops, random_init=False)
        names = dst.param_names()
        t0 = time.perf_counter()
        with open(path, "rb") as f:
            for name, shape, offset, size in index:
                f.seek(offset)
                dst.set_param(names.index(name), np.frombuffer(f.read(size), np.float32).reshape(shape))
        whole_s = time.perf_counter() - t0
        dst.close()
    print(json.dumps({"kernel": "checkpoint_load", "case": {"layers": args.layers, "dim": args.dim, "hidden": args.hidden,
                                                            "vocab": args.vocab, "tensors": len(index)},
                      "file_gb": best["file_bytes"] / 1e9, "seconds": best["seconds"],
                      "rate": best["file_bytes"] / 1e9 / best["seconds"], "unit": "GB/s",
                      "whole_tensor_sync_seconds": whole_s, "whole_tensor_sync_rate": best["file_bytes"] / 1e9 / whole_s,
                      "save_seconds": save_s, "cached_load": cached, "file": "page cache (written just before)"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
