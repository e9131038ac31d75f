#!/usr/bin/env python
"""Prefill benchmark of the decoder-only forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c3|c4|c1] ...

One step = one forward of one batch of synthetic token ids through Model::forward (the path of
`blackforge run --device cuda --from-checkpoint`). Default workload: the 2B-class decoder (vocab 32000,
d_model 2048, 16 layers, 16 heads x 128, feed-forward 5632, learned positions), precision {storage bf16,
compute bf16, accumulate fp32}, 32 sequences x 2048 tokens per GPU; weights N(0, 0.02) from a seeded
generator, ids uniform. With N GPUs (one process per GPU, launched by torchrun) the 32 sequences are split over the
ranks, 32/N each (strong scaling; `--scaling weak` gives every rank all 32): sequences are independent, so there
is no data-path collective.

Prints ONE JSON line on rank 0:
  value     tokens/s over all GPUs, ids already in HBM, device-timed (CUDA events, max over ranks)
  e2e       the same through bfb_model_forward_host with pinned HOST buffers: ids H2D and logits D2H inside
            the timed region every step
  roofline  the tcgen05 GEMM (dominant kernel): algorithmic FLOPs / event-timed duration inside the timed region
  cpu_baseline  the reference's own CPU backend (oracle/_ref) timed here on a bounded sample (N = 1 only)
Extra keys of the default workload: at 1 GPU `attention_c2` (stand-alone causal attention at its benchmark shape) and
`fp8` (the same model with compute fp8.e4m3); at 2 or more GPUs `weak` (every rank runs the whole batch) and `tp_c5`
(the 24B-class model, tensor parallel); `e2e.ceiling` puts the end-to-end figure beside what the host's links allow.
`--impl reference` times that CPU backend alone, on all host cores it can use, and prints the same line shape.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (model dims, batch per GPU, seq, precision, label)
    "c3": (dict(vocab=32000, dim=2048, layers=16, heads=16, hidden=5632, max_seq=2048), 32, 2048,
           {"storage": "bf16", "compute": "bf16", "accumulate": "fp32"},
           "2B-class decoder (vocab 32000, d 2048, 16 layers, 16x128 heads, ffn 5632) bf16 prefill"),
    "c4": (dict(vocab=32000, dim=2048, layers=16, heads=16, hidden=5632, max_seq=2048), 32, 2048,
           {"storage": "bf16", "compute": "fp8.e4m3", "accumulate": "fp32"},
           "2B-class decoder (vocab 32000, d 2048, 16 layers, 16x128 heads, ffn 5632) fp8.e4m3 prefill"),
    "c1": (dict(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32), 4, 32, None,
           "tiny decoder (vocab 256, d 64, 2 layers, 4x16 heads, ffn 256) fp32"),
    # tensor parallel: every rank runs the SAME 8 sequences on its shard of the heads, feed-forward columns and
    # logits columns; needs --gpus 2, 4 or 8 (the fp32 master weights alone are 97 GB)
    "c5": (dict(vocab=32000, dim=8192, layers=32, heads=64, hidden=28672, max_seq=4096), 8, 4096,
           {"storage": "bf16", "compute": "bf16", "accumulate": "fp32"},
           "24B-class decoder (vocab 32000, d 8192, 32 layers, 64x128 heads, ffn 28672) bf16 prefill, tensor parallel"),
}
TENSOR_PARALLEL = {"c5"}

# DRAM bytes per launch of the dominant kernel from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum),
# keyed by workload; None where no capture of that kernel has been summarised.
# c3: capture of M=32768, N=K=2048 (239.2 MB for 0.275 TFLOP, equal to A+B+C) scaled by FLOPs to the step's average
# GEMM launch (1.418 TFLOP).
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"c3": 1.233e9, "c4": None, "c1": None, "c5": None}


def lm_ops(vocab, dim, layers, heads, hidden, max_seq):
    ops, vid = [], 0

    def push(kind, **kw):
        nonlocal vid
        op = {"kind": kind, "input": vid, "output": vid + 1}
        op.update(kw)
        ops.append(op)
        vid += 1

    push("embedding", vocab=vocab, emb_dim=dim)
    push("positional_embedding", max_seq=max_seq)
    for _ in range(layers):
        push("attention", heads=heads)
        push("feedforward", hidden=hidden)
    push("linear", linear_out=vocab)
    return ops


def flops_per_token(cfg, seq):
    """Algorithmic FLOPs per token: GEMMs 2*(L*(4 d^2 + 2 d f) + d V); causal attention L*H*4*D*(S+1)/2."""
    d, f, L, V, H = cfg["dim"], cfg["hidden"], cfg["layers"], cfg["vocab"], cfg["heads"]
    gemm = 2.0 * (L * (4.0 * d * d + 2.0 * d * f) + d * V)
    attn = L * H * 4.0 * (d // H) * (seq + 1) / 2.0
    return gemm, attn


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops_burst": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 100 ms; started before the warm-up (the tool needs
    about a second to deliver its first line) and filtered to the timed window afterwards."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(device_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, t_begin: float, t_end: float):
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((stamp, float(parts[1]), float(parts[2]), float(parts[3]),
                             [n for n, v in zip(names, parts[4:8]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t_begin - 0.05 <= r[0] <= t_end + 0.05]
        window = "timed region"
        if not inside and rows:   # region shorter than the sampling period: take the samples at highest power
            inside = sorted(rows, key=lambda r: -r[3])[: max(1, len(rows) // 4)]
            window = "highest-power quarter of the run (timed region shorter than the sampling period)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no nvidia-smi samples"]}
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[0][2],
                "power_w_max": max(r[3] for r in inside), "samples": len(inside), "window": window,
                "reasons": sorted({n for r in inside for n in r[4]})}


def synth_weights(bfb, model, seed, sigma):
    """N(0, sigma) for every parameter, one PCG64 stream per parameter (seed, index)."""
    for i, _name in enumerate(model.param_names()):
        shape = model.param_shape(i)
        rng = np.random.Generator(np.random.PCG64([seed, i]))
        model.set_param(i, rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma))


def profile_read(bfb, kind):
    ms, n, work = C.c_double(), C.c_int64(), C.c_double()
    bfb.check(bfb.lib().bfb_profile_read(kind, C.byref(ms), C.byref(n), C.byref(work)))
    return ms.value, n.value, work.value


# ---------------------------------------------------------------------------------------------------------
# CPU side: the reference's own backend (oracle/_ref), bounded sample of the same layer shapes
# ---------------------------------------------------------------------------------------------------------

def cpu_sample_setup(cfg, sample_seq):
    """Returns (callable running one forward of a 1-layer, 1-sequence model with the workload's layer shapes,
    algorithmic FLOPs of that forward, kind)."""
    one = dict(cfg, layers=1, max_seq=max(sample_seq, 1))
    g, a = flops_per_token(one, sample_seq)
    flops = (g + a) * sample_seq
    from oracle import bf_oracle as O
    from oracle import ref_lib as R
    ids = O.synth_token_ids(1, sample_seq, cfg["vocab"], seed=5)
    if R.available():
        compiled = R.Compiled(O.lm_source(seq=sample_seq, **one))
        model = R.Model(compiled, 42)
        return (lambda: model.forward(ids)), flops, "reference"
    ops = O.lm_ops(**one)
    params = O.synth_params(ops, None, seed=1, sigma=0.02)
    return (lambda: O.model_forward(ops, params, ids, exact_order=True)), flops, "port"


def cpu_worker(cfg, sample_seq, steps, conn):
    try:
        run, flops, kind = cpu_sample_setup(cfg, sample_seq)
        conn.send(("ready", flops, kind))
        for _ in range(steps):
            if conn.recv() != "go":
                break
            t0 = time.perf_counter()
            run()
            conn.send(("done", time.perf_counter() - t0))
    except Exception as exc:  # pragma: no cover - reported to the parent
        conn.send(("error", repr(exc)))


def run_reference_arm(args, cfg, seq, label, precision):
    import multiprocessing as mp
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_seq = args.cpu_sample_seq
    cores = os.cpu_count() or 1
    try:
        import psutil
        by_mem = int(psutil.virtual_memory().available // (4 << 30))
    except Exception:
        by_mem = 8
    workers = max(1, min(cores, by_mem, args.cpu_workers))
    total_steps = args.warmup + args.steps
    ctx = mp.get_context("spawn")
    procs = []
    for _ in range(workers):
        parent, child = ctx.Pipe()
        p = ctx.Process(target=cpu_worker, args=(cfg, sample_seq, total_steps, child), daemon=True)
        p.start()
        procs.append((p, parent))
    flops, kind = None, "reference"
    for _p, conn in procs:
        msg = conn.recv()
        if msg[0] != "ready":
            print(json.dumps({"impl": "reference", "unavailable": f"CPU worker failed: {msg[1]}"}))
            return
        flops, kind = msg[1], msg[2]
    times = []
    for step in range(total_steps):
        t0 = time.perf_counter()
        for _p, conn in procs:
            conn.send("go")
        for _p, conn in procs:
            msg = conn.recv()
            if msg[0] != "done":
                print(json.dumps({"impl": "reference", "unavailable": f"CPU worker failed: {msg[1]}"}))
                return
        if step >= args.warmup:
            times.append(time.perf_counter() - t0)
    for p, _conn in procs:
        p.join(timeout=5)
    g, a = flops_per_token(cfg, seq)
    per_step = sum(times) / len(times)
    tokens_per_s = workers * flops / per_step / (g + a)
    sample = (f"{workers} independent processes, each one forward of a 1-layer model with the workload's layer shapes "
              f"(d {cfg['dim']}, ffn {cfg['hidden']}, vocab {cfg['vocab']}) on 1 x {sample_seq} tokens per step; "
              f"tokens/s of the full workload extrapolated by algorithmic FLOPs ({(g + a) / 1e9:.3f} GFLOP/token)")
    line = {
        "impl": "reference", "metric": "prefill tokens/s", "value": tokens_per_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True,
        "scaling": "strong" if (args.gpus > 1 and args.scaling != "weak") or args.workload in TENSOR_PARALLEL else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": label, "seq_len": seq, "precision": precision or "fp32 (no precision block)"},
        "cpu_baseline": {"value": tokens_per_s, "unit": "tokens/s", "cores": workers, "kind": kind, "sample": sample,
                         "host_cores": cores, "gflops": workers * flops / per_step / 1e9},
        "e2e": {"value": tokens_per_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_decode(args, bfb, launch, torch, model, cfg, batch, ids, precision, label, rank, world, local, dev):
    """Generation with key/value caches (Model::forwardIncremental): prompt untimed, then K single-token steps.
    Bound by HBM: every step streams all GEMM weights and the whole key/value cache once."""
    context = min(args.context, cfg["max_seq"] - args.steps - max(args.warmup, 1))
    if context < 1:
        raise SystemExit("--context, --warmup and --steps do not fit in the positional table")
    prompt = bfb.DeviceBuffer.from_numpy(np.ascontiguousarray(ids[:, :context]))
    step_ids = [bfb.DeviceBuffer.from_numpy(np.ascontiguousarray(ids[:, context + i:context + i + 1]))
                for i in range(max(args.warmup, 1) + args.steps)]
    def prime():
        model.reset_generation()
        out, _ = model.forward_incremental_device(prompt.ptr, (batch, context), trusted=True)
        out.free()
        for i in range(max(args.warmup, 1)):
            out, _ = model.forward_incremental_device(step_ids[i].ptr, (batch, 1), trusted=True)
            out.free()
        torch.cuda.synchronize()

    def steps():
        for i in range(args.steps):
            out, _ = model.forward_incremental_device(step_ids[max(args.warmup, 1) + i].ptr, (batch, 1), trusted=True)
            out.free()

    sampler = ClockSampler(local) if rank == 0 else None
    prime()
    bfb.lib().bfb_launch_count(1)
    launch.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall_begin = time.time()
    start.record()
    steps()
    stop.record()
    torch.cuda.synchronize()
    wall_end = time.time()
    launch.barrier()
    elapsed_ms = launch.max_over_ranks(start.elapsed_time(stop), dev if world > 1 else None)
    clocks = sampler.stop(wall_begin, wall_end) if sampler else None
    launches = bfb.lib().bfb_launch_count(0)
    # per-kernel times from a second pass over the same positions: the events around every launch would otherwise sit
    # between the kernels of the timed steps (a step is some 180 short launches) and keep them from overlapping
    prime()
    bfb.lib().bfb_profile_reset()
    bfb.lib().bfb_profile_enable(1)
    steps()
    torch.cuda.synchronize()
    bfb.lib().bfb_profile_enable(0)
    kernels = {}
    for name, kind in (("gemm_tcgen05", 0), ("attention_tcgen05", 1), ("rmsnorm", 2), ("embed_pos", 3), ("cast", 4)):
        ms, n, work = profile_read(bfb, kind)
        if n:
            kernels[name] = {"ms_total": ms, "launches": n, "ms_per_step": ms / args.steps,
                             "measured": "separate pass with events around each launch"}
    if world > 1:
        launch.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    ms_per_step = elapsed_ms / args.steps
    d, f, v, layers = cfg["dim"], cfg["hidden"], cfg["vocab"], cfg["layers"]
    wbytes = 1 if (precision or {}).get("compute") == "fp8.e4m3" else 2
    weight_bytes = (layers * (4 * d * d + 2 * d * f) + d * v) * wbytes
    mean_ctx = context + max(args.warmup, 1) + (args.steps - 1) / 2.0
    cache_bytes = 2 * layers * batch * mean_ctx * d * 2          # K and V, bf16, read once per step
    peaks = measured_peaks()
    achieved = (weight_bytes + cache_bytes) / (ms_per_step / 1e3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": world * batch / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": (precision or {}).get("compute", "f32"), "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)",
        "config": {"workload": label + ", generation with key/value caches", "batch_per_gpu": batch,
                   "context": context, "new_tokens_per_step": 1, "precision": precision,
                   "l2": "every step streams GBs of weights and cache: far beyond the 126 MB L2, no flush needed"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                     "bytes_per_step": {"weights": weight_bytes, "kv_cache": cache_bytes},
                     "peak_source": "of " + peaks["source"] + " (copy bandwidth)"},
        "kernels": kernels, "gpu_launches": int(launches), "clocks": clocks,
    }
    print(json.dumps(line))


def cpu_baseline_inline(cfg, seq, sample_seq):
    """Single-thread reference CPU backend on the bounded sample (the reference has no threading)."""
    run, flops, kind = cpu_sample_setup(cfg, sample_seq)
    t0 = time.perf_counter()
    run()
    dt = time.perf_counter() - t0
    g, a = flops_per_token(cfg, seq)
    return {"value": flops / dt / (g + a), "unit": "tokens/s", "cores": 1, "kind": kind, "host_cores": os.cpu_count(),
            "gflops": flops / dt / 1e9, "seconds": dt,
            "sample": (f"one forward of a 1-layer model with the workload's layer shapes on 1 x {sample_seq} tokens, "
                       f"single thread; tokens/s of the full workload extrapolated by algorithmic FLOPs")}


# ---------------------------------------------------------------------------------------------------------
# measurement pieces of the default arm
# ---------------------------------------------------------------------------------------------------------

KERNEL_KINDS = (("gemm_tcgen05", 0), ("attention_tcgen05", 1), ("rmsnorm", 2), ("embed_pos", 3), ("cast", 4))


class Ctx:
    """What every measurement needs: the binding, rank plumbing and the current device."""

    def __init__(self, bfb, launch, torch, rank, world, local):
        self.bfb, self.launch, self.torch = bfb, launch, torch
        self.rank, self.world, self.local = rank, world, local
        self.dev = torch.device("cuda", local)

    def max_ms(self, ms):
        return self.launch.max_over_ranks(ms, self.dev if self.world > 1 else None)


def build_model(ctx, cfg, precision, tensor_parallel, seed, tp_groups=2, tp_reserved_sms=0):
    bfb = ctx.bfb
    model = bfb.Model(lm_ops(**cfg), precision=precision, random_init=False)
    if tensor_parallel:
        model.set_tensor_parallel(ctx.rank, ctx.world)
        model.set_tensor_parallel_overlap(tp_groups, tp_reserved_sms if tp_groups > 1 else 0)
        # weights drawn on the device (N(0, 0.01), the same full matrices whatever the split); the fp32 copies of
        # the GEMM weights are dropped once the first forward has converted them
        for i, _name in enumerate(model.param_names()):
            model.fill_param_normal(i, seed * 1000003 + i, 0.01)
    else:
        synth_weights(bfb, model, seed, 0.02)
    return model


def draw_ids(cfg, batch, seq, seed, stream_id):
    rng = np.random.Generator(np.random.PCG64([seed, 7919 + stream_id]))
    return rng.integers(0, cfg["vocab"], size=(batch, seq)).astype(np.float32)


def time_device_steps(ctx, model, d_ids, shape, steps, warmup, release_masters=False, sample_clocks=False):
    """W warm-up and K timed forwards with the ids resident in HBM: CUDA events on the launching stream, barrier and
    synchronize on both sides, max over ranks; per-kernel device times from the library's own events."""
    bfb, torch = ctx.bfb, ctx.torch

    def step():
        out, oshape = model.forward_device(d_ids.ptr, shape, trusted=True)
        out.free()   # back to the pool: the next step reuses the same memory
        return oshape

    sampler = ClockSampler(ctx.local) if (sample_clocks and ctx.rank == 0) else None
    out_shape = None
    for i in range(max(warmup, 1)):
        out_shape = step()
        if i == 0 and release_masters:
            torch.cuda.synchronize()
            model.release_master_weights()
    torch.cuda.synchronize()
    bfb.lib().bfb_profile_reset()
    bfb.lib().bfb_profile_enable(1)
    bfb.lib().bfb_launch_count(1)
    ctx.launch.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall_begin = time.time()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    wall_end = time.time()
    ctx.launch.barrier()
    elapsed_ms = ctx.max_ms(start.elapsed_time(stop))
    clocks = sampler.stop(wall_begin, wall_end) if sampler else None
    launches = bfb.lib().bfb_launch_count(0)
    bfb.lib().bfb_profile_enable(0)
    kernels = {}
    for name, kind in KERNEL_KINDS:
        ms, n, work = profile_read(bfb, kind)
        if n:
            secs = ms / 1e3
            k = {"ms_total": ms, "launches": n, "work": work, "share_of_step": ms / elapsed_ms}
            if name in ("gemm_tcgen05", "attention_tcgen05"):
                k["tflops"] = work / secs / 1e12
            else:
                k["gbs"] = work / secs / 1e9
            kernels[name] = k
    bfb.lib().bfb_profile_reset()
    return {"ms_per_step": elapsed_ms / steps, "elapsed_ms": elapsed_ms, "kernels": kernels, "launches": int(launches),
            "clocks": clocks, "out_shape": out_shape}


def time_e2e(ctx, model, ids, out_shape, steps, precision, tokens_global):
    """The same forward through the host-buffer API: pinned host ids in, pinned host logits out, both copies inside
    the timed region of every step."""
    bfb, torch = ctx.bfb, ctx.torch
    out_elems = int(np.prod(out_shape))
    h_ids = torch.from_numpy(ids).pin_memory()
    h_out = torch.empty(out_elems, dtype=torch.float32).pin_memory()
    shape_arr = (C.c_int64 * 2)(*ids.shape)
    oshape, orank = (C.c_int64 * 8)(), C.c_int32()

    def timed(fn):
        fn()
        ctx.launch.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        torch.cuda.synchronize()
        ctx.launch.barrier()
        return ctx.max_ms(s.elapsed_time(e)) / steps

    ms = timed(lambda: bfb.check(bfb.lib().bfb_model_forward_host(model._h, h_ids.data_ptr(), shape_arr, 2,
                                                                   h_out.data_ptr(), oshape, C.byref(orank))))
    # bytes the call itself booked for its copies: under storage bf16 part of the logits may cross the link as
    # 2-byte bf16 and be widened to the caller's fp32 buffer by host threads
    h2d_bytes, d2h_bytes = bfb.host_transfer_bytes()
    e2e = {"value": tokens_global / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms,
           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
           "result_bytes_per_step": out_elems * 4, "steps": steps,
           "api": "bfb_model_forward_host (fromHost -> Model::forward -> toHost), pinned host buffers"}
    del h_out
    # the same pipeline handing the logits to the host as bf16 (bfb_model_forward_host_bf16): not the reference's
    # fp32 contract, reported beside it because it is what keeps several GPUs from saturating one host
    if (precision or {}).get("storage") == "bf16":
        h_out16 = torch.empty(out_elems, dtype=torch.int16).pin_memory()
        ms16 = timed(lambda: bfb.check(bfb.lib().bfb_model_forward_host_bf16(
            model._h, h_ids.data_ptr(), shape_arr, 2, h_out16.data_ptr(), oshape, C.byref(orank))))
        e2e["bf16_result"] = {"value": tokens_global / (ms16 / 1e3), "unit": "tokens/s", "ms_per_step": ms16,
                              "d2h_bytes_per_step": bfb.host_transfer_bytes()[1],
                              "api": "bfb_model_forward_host_bf16 (logits stay bf16 on the host)"}
        del h_out16
    return e2e


def d2h_probe(ctx, nbytes=1 << 30, repeats=3):
    """Device-to-pinned-host copies of `nbytes` issued by every rank at the same time: what this host takes in from
    its GPUs together (GB/s over all ranks, max-over-ranks time), the ceiling of any end-to-end figure."""
    torch = ctx.torch
    src = torch.empty(nbytes, dtype=torch.uint8, device=ctx.dev)
    dst = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dst.copy_(src, non_blocking=True)
    torch.cuda.synchronize()
    ctx.launch.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(repeats):
        dst.copy_(src, non_blocking=True)
    e.record()
    torch.cuda.synchronize()
    ctx.launch.barrier()
    ms = ctx.max_ms(s.elapsed_time(e)) / repeats
    return {"aggregate_gbs": ctx.world * nbytes / (ms / 1e3) / 1e9, "per_rank_gbs": nbytes / (ms / 1e3) / 1e9,
            "bytes_per_rank": nbytes, "ranks": ctx.world}


def attention_config2(ctx, peaks, iters=20, warmup=3):
    """BASELINE config 2: stand-alone causal attention, Q/K/V bf16 [16, 16 heads, 2048, 128] i.i.d. N(0,1), scale
    1/sqrt(128); CUDA events, L2 flushed between iterations (the operands are 4 x 134 MB, about the size of L2)."""
    bfb, torch = ctx.bfb, ctx.torch
    lib = bfb.lib()
    batch, heads, seq, hd = 16, 16, 2048, 128
    dim = heads * hd
    n = batch * seq * dim

    def rand_bf16(seed):
        g = torch.Generator(device=ctx.dev)
        g.manual_seed(seed)
        t = torch.randn(n, device=ctx.dev, dtype=torch.float32, generator=g)
        buf = bfb.DeviceBuffer(n * 2)
        bfb.check(lib.bfb_cast(t.data_ptr(), bfb.F32, buf.ptr, bfb.BF16, n, 1.0, None, None))
        torch.cuda.synchronize()
        return buf

    q, k, v = rand_bf16(11), rand_bf16(12), rand_bf16(13)
    out = bfb.DeviceBuffer(n * 2)
    status = bfb.DeviceBuffer.zeros(4)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=ctx.dev)

    def run():
        bfb.check(lib.bfb_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, None, None, bfb.BF16, batch, seq, seq, heads, hd,
                                        dim, dim, dim, dim, float(hd ** -0.5), 0, 1, status.ptr, None))

    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    code = int(status.to_numpy(np.int32, (1,))[0])
    ms = statistics.median(times)
    flops = 4.0 * hd * batch * heads * seq * (seq + 1) / 2.0
    tflops = flops / (ms / 1e3) / 1e12
    # the backward of the same problem (the training-side kernel): statistics kernel, zero fill of dQ and the tcgen05
    # kernel, from the forward's output and row statistics
    backward = None
    try:
        rows = batch * heads * seq
        g = rand_bf16(14)
        m_, l_, scratch = bfb.DeviceBuffer(rows * 4), bfb.DeviceBuffer(rows * 4), bfb.DeviceBuffer(rows * 8)
        grads = [bfb.DeviceBuffer(n * 4) for _ in range(3)]
        bfb.check(lib.bfb_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, m_.ptr, l_.ptr, bfb.BF16, batch, seq, seq, heads, hd,
                                        dim, dim, dim, dim, float(hd ** -0.5), 0, 1, status.ptr, None))

        def run_bwd():
            bfb.check(lib.bfb_attention_bwd(g.ptr, q.ptr, k.ptr, v.ptr, out.ptr, m_.ptr, l_.ptr, grads[0].ptr, grads[1].ptr,
                                            grads[2].ptr, scratch.ptr, bfb.BF16, batch, seq, seq, heads, hd, dim, dim, dim,
                                            dim, float(hd ** -0.5), 0, 1, status.ptr, None))
        for _ in range(warmup):
            run_bwd()
        torch.cuda.synchronize()
        btimes = []
        for _ in range(max(5, iters // 2)):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run_bwd()
            e.record()
            torch.cuda.synchronize()
            btimes.append(s.elapsed_time(e))
        bms = statistics.median(btimes)
        backward = {"kernel": "attentionBackwardTcKernel (tcgen05, keys on the tensor-memory lanes, dQ added by TMA)",
                    "ms": bms, "tflops": 2.5 * flops / (bms / 1e3) / 1e12, "flops": "causal: five products of 2*D per visible pair",
                    "device_status": int(status.to_numpy(np.int32, (1,))[0])}
        for b in [g, m_, l_, scratch] + grads:
            b.free()
    except Exception as exc:   # the forward figure stands without it
        backward = {"error": repr(exc)}
    for b in (q, k, v, out, status):
        b.free()
    return {"workload": "causal attention forward, bf16 [16, 16, 2048, 128], fp32 online softmax (BASELINE config 2)",
            "backward": backward,
            "kernel": "attentionTcKernel (tcgen05, S/P/O in tensor memory, TMA-fed)", "ms": ms, "ms_min": min(times),
            "tflops": tflops, "flops": "causal: 4*D per visible (query, key) pair", "iters": iters,
            "frac_of_burst": tflops / peaks["tflops_burst"], "frac_of_sustained": tflops / peaks["tflops_sustained"],
            "frac_of_nominal_2250": tflops / 2250.0, "peak_source": "of " + peaks["source"] + " (cuBLAS bf16)",
            "l2": "256 MiB written between iterations", "device_status": code}


NOMINAL_FP8_TFLOPS = 4500.0


def fp8_config4(ctx, args, peaks, bf16_ms):
    """BASELINE config 4 beside the headline: the same model with compute fp8.e4m3, a few steps."""
    cfg, batch, seq, precision, label = WORKLOADS["c4"]
    model = build_model(ctx, dict(cfg), precision, False, args.seed)
    ids = draw_ids(cfg, batch, seq, args.seed, ctx.rank)
    d_ids = ctx.bfb.DeviceBuffer.from_numpy(ids)
    m = time_device_steps(ctx, model, d_ids, ids.shape, steps=max(3, min(args.steps, 5)), warmup=3)
    d_ids.free()
    model.close()
    ctx.bfb.check(ctx.bfb.lib().bfb_pool_trim())
    g, a = flops_per_token(cfg, seq)
    tokens = batch * seq
    res = {"workload": label, "tokens_per_s": tokens / (m["ms_per_step"] / 1e3), "ms_per_step": m["ms_per_step"],
           "speedup_vs_bf16_step": bf16_ms / m["ms_per_step"] if bf16_ms else None,
           "model_tflops": (g + a) * tokens / (m["ms_per_step"] / 1e3) / 1e12, "gpu_launches": m["launches"],
           "kernels": m["kernels"], "parity": "unpinned (the reference has no fp8 implementation)"}
    k = m["kernels"].get("gemm_tcgen05")
    if k:
        res["gemm_tflops"] = k["tflops"]
        res["gemm_frac_of_nominal_4500"] = k["tflops"] / NOMINAL_FP8_TFLOPS
        res["peak_note"] = ("no fp8 peak was measured on this pool: the fraction is of the NOMINAL dense fp8 figure "
                            f"({NOMINAL_FP8_TFLOPS:.0f} TFLOP/s); the measured bf16 cuBLAS peaks are "
                            f"{peaks['tflops_burst']:.0f} burst / {peaks['tflops_sustained']:.0f} sustained")
    return res


def tensor_parallel_config5(ctx, args, steps=3, warmup=2):
    """BASELINE config 5 on this many GPUs: the 24B-class model, heads / feed-forward columns / logits columns
    sharded, NCCL all-reduces hidden behind the next sequence group's kernels. Every rank runs the same 8 x 4096
    tokens."""
    bfb, launch = ctx.bfb, ctx.launch
    cfg, batch, seq, precision, label = WORKLOADS["c5"]
    ident = launch.broadcast_bytes(bfb.tp_unique_id() if ctx.rank == 0 else b"", 128, 0, ctx.dev)
    bfb.tp_init(ident, ctx.rank, ctx.world)
    model = build_model(ctx, dict(cfg), precision, True, args.seed, args.tp_groups, args.tp_reserved_sms)
    ids = draw_ids(cfg, batch, seq, args.seed, 0)    # the same sequences on every rank
    d_ids = bfb.DeviceBuffer.from_numpy(ids)
    m = time_device_steps(ctx, model, d_ids, ids.shape, steps=steps, warmup=warmup, release_masters=True)
    d_ids.free()
    model.close()
    bfb.tp_destroy()
    bfb.check(bfb.lib().bfb_pool_trim())
    g, a = flops_per_token(cfg, seq)
    tokens = batch * seq
    kern = m["kernels"]
    busy = sum(k["ms_total"] for k in kern.values()) / steps
    res = {"workload": label, "tokens_per_s": tokens / (m["ms_per_step"] / 1e3), "ms_per_step": m["ms_per_step"],
           "model_tflops_per_gpu": (g + a) * tokens / (m["ms_per_step"] / 1e3) / 1e12 / ctx.world,
           "gemm_tflops": kern.get("gemm_tcgen05", {}).get("tflops"),
           "attention_tflops": kern.get("attention_tcgen05", {}).get("tflops"),
           # what the step takes beyond its own kernels back to back on the compute stream: all-reduce time that
           # is NOT hidden, plus launch gaps
           "allreduce_exposed_ms": max(0.0, m["ms_per_step"] - busy), "kernel_ms_per_step": busy,
           "allreduces_per_step": 2 * cfg["layers"] * max(args.tp_groups, 1),
           "allreduce_bytes_per_step": 2 * cfg["layers"] * tokens * cfg["dim"] * 2,
           "sequence_groups": args.tp_groups, "steps": steps, "warmup": warmup, "gpu_launches": m["launches"],
           "scaling": "strong (the same batch on 2, 4 or 8 GPUs)"}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="auto", choices=["auto", "strong", "weak"],
                    help="batch-sharded workloads on N GPUs: strong = the workload's batch split over the ranks "
                         "(32 -> 32/N sequences per GPU; the default), weak = the whole batch on every rank")
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (default: the workload's)")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (invalid as a headline number)")
    ap.add_argument("--e2e-steps", type=int, default=-1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra keys (attention_c2 and fp8 at 1 GPU; weak and tp_c5 at 2 or more)")
    ap.add_argument("--cpu-sample-seq", type=int, default=32,
                    help="tokens per worker and step of the reference arm's bounded sample")
    ap.add_argument("--cpu-baseline-seq", type=int, default=192,
                    help="tokens of the single-thread cpu_baseline sample of the default arm (about 11 s)")
    ap.add_argument("--cpu-workers", type=int, default=32)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--tp-groups", type=int, default=2,
                    help="tensor-parallel workloads: sequence groups whose all-reduces overlap the next group's GEMMs (1: none)")
    ap.add_argument("--tp-reserved-sms", type=int, default=0,
                    help="SMs the persistent kernels leave to the overlapped collective")
    ap.add_argument("--decode", action="store_true",
                    help="measure key/value-cache generation instead of prefill: a prompt of --context tokens per "
                         "sequence (untimed), then --steps single-token steps for the whole batch")
    ap.add_argument("--context", type=int, default=1920)
    args = ap.parse_args()

    cfg, batch, seq, precision, label = WORKLOADS[args.workload]
    cfg = dict(cfg)
    reduced = False
    if args.batch:
        batch, reduced = args.batch, True
    if args.seq:
        seq, reduced = args.seq, True
    if args.layers:
        cfg["layers"], reduced = args.layers, True
    if reduced:
        label += " [REDUCED: not the headline configuration]"

    if args.impl == "reference":
        run_reference_arm(args, cfg, seq, label, precision)
        return

    import torch
    import blackforge_b200 as bfb
    from blackforge_b200 import launch

    rank, world, local = launch.env_ranks()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU fallback")
    torch.cuda.set_device(local)
    bfb.check(bfb.lib().bfb_set_device(local))
    if world > 1:
        launch.init_process_group("nccl")
    ctx = Ctx(bfb, launch, torch, rank, world, local)
    dev = ctx.dev

    tensor_parallel = args.workload in TENSOR_PARALLEL
    if tensor_parallel and world < 2:
        raise SystemExit(f"workload {args.workload} is tensor parallel: launch it on 2, 4 or 8 GPUs")
    # batch-sharded workloads: strong scaling splits the workload's batch over the ranks, weak gives every rank all of it
    scaling = "strong" if tensor_parallel else (args.scaling if args.scaling != "auto" else ("strong" if world > 1 else "weak"))
    global_batch = batch
    if tensor_parallel:
        batch_per_gpu = batch
    elif scaling == "strong" and world > 1:
        if batch % world:
            raise SystemExit(f"strong scaling needs the batch ({batch}) to divide by --gpus ({world})")
        batch_per_gpu = batch // world
    else:
        batch_per_gpu, global_batch = batch, batch * world

    # ---- model and inputs --------------------------------------------------------------------------------
    if tensor_parallel:
        ident = launch.broadcast_bytes(bfb.tp_unique_id() if rank == 0 else b"", 128, 0, dev)
        bfb.tp_init(ident, rank, world)
    model = build_model(ctx, cfg, precision, tensor_parallel, args.seed, args.tp_groups, args.tp_reserved_sms)
    # batch-sharded ranks draw their own sequences; tensor-parallel ranks must all see the same ones
    ids = draw_ids(cfg, batch_per_gpu, seq, args.seed, 0 if tensor_parallel else rank)
    d_ids = bfb.DeviceBuffer.from_numpy(ids)
    tokens_global = global_batch * seq
    if args.decode:
        run_decode(args, bfb, launch, torch, model, cfg, batch_per_gpu, ids, precision, label, rank, world, local, dev)
        return

    # ---- timed region: ids in HBM, CUDA events on the launching stream ---------------------------------------
    m = time_device_steps(ctx, model, d_ids, ids.shape, args.steps, args.warmup, release_masters=tensor_parallel,
                          sample_clocks=True)
    ms_per_step, kernels, elapsed_ms = m["ms_per_step"], m["kernels"], m["elapsed_ms"]
    value = tokens_global / (ms_per_step / 1e3)

    # ---- end to end through the host-buffer API: ids H2D + logits D2H inside the timed region ---------------
    e2e = None
    e2e_steps = args.steps if args.e2e_steps < 0 else args.e2e_steps
    if e2e_steps > 0:
        e2e = time_e2e(ctx, model, ids, m["out_shape"], e2e_steps, precision, tokens_global)
        probe = d2h_probe(ctx)
        bytes_per_token = e2e["d2h_bytes_per_step"] * (1 if tensor_parallel else world) / tokens_global
        link_rate = probe["aggregate_gbs"] * 1e9 / bytes_per_token
        e2e["ceiling"] = {"value": min(value, link_rate), "unit": "tokens/s",
                          "formula": "min(device-timed tokens/s, aggregate pinned D2H GB/s of this host / result bytes per token)",
                          "device_tokens_per_s": value, "d2h_aggregate_gbs": probe["aggregate_gbs"],
                          "d2h_per_rank_gbs": probe["per_rank_gbs"], "d2h_bytes_per_token": bytes_per_token,
                          "link_tokens_per_s": link_rate, "e2e_over_ceiling": e2e["value"] / min(value, link_rate),
                          "probe": f"{probe['bytes_per_rank'] >> 20} MiB device -> pinned host on all {world} rank(s) at once"}

    # ---- extra keys: the other halves of the headline metric --------------------------------------------------
    peaks = measured_peaks()
    extras = {}
    headline = args.workload == "c3" and not reduced and not args.no_extras
    if headline and world > 1 and scaling == "strong":
        # the weak-scaling figure beside it: every rank runs the whole 32 x 2048 batch
        w_ids = draw_ids(cfg, batch, seq, args.seed, rank)
        w_d = bfb.DeviceBuffer.from_numpy(w_ids)
        wm = time_device_steps(ctx, model, w_d, w_ids.shape, steps=3, warmup=2)
        w_d.free()
        extras["weak"] = {"value": world * batch * seq / (wm["ms_per_step"] / 1e3), "unit": "tokens/s",
                          "ms_per_step": wm["ms_per_step"], "batch_per_gpu": batch, "global_batch": batch * world,
                          "steps": 3, "warmup": 2, "scaling": "weak"}
    d_ids.free()
    model.close()
    bfb.check(bfb.lib().bfb_pool_trim())
    if tensor_parallel:
        bfb.tp_destroy()
    if headline and world == 1:
        for key, fn in (("attention_c2", lambda: attention_config2(ctx, peaks)),
                        ("fp8", lambda: fp8_config4(ctx, args, peaks, ms_per_step))):
            try:
                extras[key] = fn()
            except Exception as exc:   # an extra key must not cost the headline line
                extras[key] = {"error": repr(exc)}
    if headline and world > 1:
        try:
            extras["tp_c5"] = tensor_parallel_config5(ctx, args)
        except Exception as exc:
            extras["tp_c5"] = {"error": repr(exc)}

    if world > 1:
        launch.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return

    # ---- roofline of the dominant kernel ---------------------------------------------------------------------
    g_flops, a_flops = flops_per_token(cfg, seq)
    roofline = None
    if "gemm_tcgen05" in kernels:
        k = kernels["gemm_tcgen05"]
        fp8 = (precision or {}).get("compute") == "fp8.e4m3"
        peak = NOMINAL_FP8_TFLOPS if fp8 else peaks["tflops_sustained"]
        roofline = {"kernel": "gemmPairKernel (tcgen05 cta_group::2, 256x256 tiles per CTA pair, TMA-fed, TMEM accumulators)",
                    "bound": "tensor", "achieved": k["tflops"], "peak": peak, "unit": "TFLOP/s", "frac": k["tflops"] / peak,
                    "peak_source": ("of NOMINAL dense fp8 (no fp8 peak was measured on this pool)" if fp8 else
                                    f"of {peaks['source']} (sustained cuBLAS bf16)"),
                    "launches": k["launches"], "avg_launch_ms": k["ms_total"] / k["launches"],
                    "share_of_step": k["ms_total"] / elapsed_ms,
                    "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(args.workload)}
    # per GPU: a tensor-parallel rank does 1/world of the batch's arithmetic
    model_tflops = (g_flops + a_flops) * tokens_global / (ms_per_step / 1e3) / 1e12 / world

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_baseline_inline(cfg, seq, args.cpu_baseline_seq)
        except Exception as exc:
            cpu = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "unavailable", "sample": repr(exc)}

    line = {
        "metric": "prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": scaling,
        "vs_baseline": None, "dtype": "bf16" if (precision or {}).get("compute") == "bf16" else
        ("fp8.e4m3" if (precision or {}).get("compute") == "fp8.e4m3" else "f32"),
        "data": f"synthetic (seeded uniform token ids, N(0,{'0.01' if tensor_parallel else '0.02'}) weights)",
        "config": {"workload": label, "global_batch": global_batch, "batch_per_gpu": batch_per_gpu, "seq_len": seq,
                   "precision": precision,
                   "parallelism": (f"tensor-parallel x{world}: heads, feed-forward columns and logits columns sharded, "
                                   "NCCL all-reduce after the out-projection and the feed-forward down-projection"
                                   + (f", {args.tp_groups} sequence groups: one group's all-reduce runs beside the next "
                                      f"group's kernels, whose GEMMs draw their tiles dynamically ({args.tp_reserved_sms} SMs left free)" if args.tp_groups > 1 else "")
                                   if tensor_parallel else
                                   f"batch-sharded x{world} ({batch_per_gpu} sequences per GPU), no data-path collective"),
                   "l2": "per-step working set (weights and activations, GBs) far exceeds the 126 MB L2; no flush needed",
                   "flops_per_token": g_flops + a_flops},
        "model_tflops": model_tflops,
        "model_frac_of_peak": {"measured_sustained": model_tflops / peaks["tflops_sustained"],
                               "nominal_2250": model_tflops / 2250.0},
        "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": m["launches"],
        "clocks": m["clocks"], "peaks": peaks,
    }
    line.update(extras)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
