"""Builds blackforge_b200/libbfb200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m blackforge_b200.build [--force] [--verbose]

Objects go to blackforge_b200/_build/. The library links only the CUDA runtime; the tensor-map
encoder comes from the driver at run time and NCCL is opened with dlopen when tensor parallelism is
requested.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(HERE, "libbfb200.so")

SOURCES = [
    "pool.cu",
    "elementwise.cu",
    "quantize.cu",
    "gemm_simt.cu",
    "gemm_tc.cu",
    "gemm_tc2.cu",
    "gemm_skinny.cu",
    "attention_simt.cu",
    "attention_tc.cu",
    "attention_bwd.cu",
    "attention_decode.cu",
    "selftest.cu",
    "capi.cu",
    "host/ops.cpp",
    "host/model.cpp",
    "host/tp.cpp",
    "host/widen.cpp",
    "host/watchdog.cpp",
    "host/checkpoint.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libbfb200.so")
    return cand


def _headers():
    out = []
    for root, _dirs, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".hpp", ".cuh", ".h"))]
    out.append(os.path.join(os.path.dirname(HERE), "include", "bfb200.h"))
    return out


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    os.makedirs(BUILD_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    jobs = []
    objects = []
    for src in sources:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(BUILD_DIR, src.replace("/", "_") + ".o")
        objects.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-x", "cu", "-c", src_path, "-o", obj]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return src, proc

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for src, proc in pool.map(run, jobs):
                if verbose or proc.returncode != 0 or ptxas_info:
                    sys.stderr.write(f"--- {src}\n{proc.stdout}{proc.stderr}\n")
                if proc.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src}")
    if jobs or force or _stale(LIB_PATH, objects):
        cmd = [nvcc, "-shared", "-o", LIB_PATH] + objects + ["-lcudart", "-ldl", "-Xlinker", "--no-undefined"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("linking libbfb200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
