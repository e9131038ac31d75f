"""C++ callers of the library, run as programs on the GPU:

* tests/cpp/ops_mirror_test.cpp — the operator-level C++ mirror (namespace bfb200) used directly: the bf16 / e4m3
  operator forms and the DeviceTensor mechanics that Model::forward does not go through. Compiled here with g++
  (it needs only the repository's own header and library).
* oracle/_ref/dropin_reference_caller — caller code written against the REFERENCE's headers (the way its own CUDA
  tests are written), linked with the drop-in translation unit blackforge_b200/dropin/blackforge_backend_cuda.cpp
  and libbfb200.so in place of the reference's CUDA sources. Built by `make -C oracle dropin` where the reference's
  headers exist; skipped where that was not done.
"""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(cmd, **kw):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, **kw)
    print(proc.stdout)
    return proc


def test_operator_level_cpp_mirror(gpu, tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++ on this machine")
    cuda_inc, cuda_lib = "/usr/local/cuda/include", "/usr/local/cuda/lib64"
    exe = tmp_path / "ops_mirror_test"
    lib_dir = os.path.join(ROOT, "blackforge_b200")
    build = run([gxx, "-std=c++17", "-O1", "-I" + cuda_inc, os.path.join(ROOT, "tests", "cpp", "ops_mirror_test.cpp"), "-o", str(exe),
                 "-L" + lib_dir, "-lbfb200", "-L" + cuda_lib, "-lcudart", "-Wl,-rpath," + lib_dir, "-Wl,-rpath," + cuda_lib])
    assert build.returncode == 0, build.stdout
    proc = run([str(exe)])
    assert proc.returncode == 0 and "all checks passed" in proc.stdout, proc.stdout


def test_reference_style_caller_runs_on_the_drop_in(gpu, tmp_path):
    exe = os.path.join(ROOT, "oracle", "_ref", "dropin_reference_caller")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/dropin_reference_caller not built (make -C oracle dropin needs the reference's headers)")
    proc = run([exe, str(tmp_path)])
    assert proc.returncode == 0 and "all checks passed" in proc.stdout, proc.stdout
