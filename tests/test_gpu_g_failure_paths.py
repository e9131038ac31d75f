"""Failure paths on the device, taken on purpose in forms that cannot harm it: a bounded wait that is made to run
out (short limit, a barrier nobody arrives on; the kernel returns a status, nothing traps), and an allocation
failure injected on the host. After each, the same context keeps working."""
import ctypes as C

import numpy as np
import pytest

from oracle import bf_oracle as O

pytestmark = pytest.mark.gpu


def small_gemm_ok(gpu):
    rng = np.random.default_rng(5)
    a = O.round_bf16(rng.standard_normal((256, 128)).astype(np.float32))
    w = O.round_bf16(rng.standard_normal((256, 128)).astype(np.float32))
    da, dw = gpu.upload(a, gpu.BF16), gpu.upload(w, gpu.BF16)
    dc = gpu.DeviceBuffer(256 * 256 * 4)
    status = gpu.DeviceBuffer.zeros(4)
    gpu.check(gpu.lib().bfb_gemm(da.ptr, dw.ptr, dc.ptr, 256, 256, 128, gpu.BF16, gpu.B_NK, gpu.F32, gpu.EPI["none"], None,
                                 None, 1.0, None, 0, status.ptr, None))
    gpu.sync()
    got = dc.to_numpy(np.float32, (256, 256))
    assert int(status.to_numpy(np.int32, (1,))[0]) == 0
    assert np.max(np.abs(got - a.astype(np.float64) @ w.astype(np.float64).T)) <= 1e-3
    for b in (da, dw, dc, status):
        b.free()


def test_a_bounded_wait_that_runs_out_returns_timeout_and_leaves_the_context_usable(gpu):
    lib = gpu.lib()
    observed = (C.c_int32 * 3)()
    status = lib.bfb_selftest_bounded_wait(1_000_000, observed, None)       # 1 ms
    assert status == gpu.TIMEOUT
    assert b"bounded wait" in lib.bfb_last_error()
    # neither wait was satisfied; the second role, whose own limit is 1.5 s, left because of the abort flag
    assert observed[0] == 0 and observed[1] == 0
    assert observed[2] < 500_000, f"the second role waited {observed[2]} us"
    with pytest.raises(gpu.RuntimeFailure) as err:
        gpu.check(lib.bfb_selftest_bounded_wait(200_000, None, None))
    assert err.value.status == gpu.TIMEOUT
    # the context is intact: the next tensor-core GEMM on the same stream gives the right numbers
    small_gemm_ok(gpu)


def pool_stats(gpu):
    cached, live = C.c_size_t(0), C.c_size_t(0)
    gpu.check(gpu.lib().bfb_pool_stats(C.byref(cached), C.byref(live)))
    return cached.value, live.value


def test_an_injected_allocation_failure_is_reported_and_leaks_nothing(gpu):
    lib = gpu.lib()
    cfg = dict(vocab=256, dim=256, layers=2, heads=2, hidden=512, max_seq=64)
    ops = O.lm_ops(**cfg)
    model = gpu.Model(ops, precision={"storage": "bf16", "compute": "bf16"}, seed=3)
    ids = O.synth_token_ids(2, 64, cfg["vocab"], seed=4)
    want = model.forward_host(ids)           # first pass: weights converted, scratch buffers in place
    _, live_before = pool_stats(gpu)
    failures = 0
    for nth in (1, 2, 3, 5):
        gpu.check(lib.bfb_pool_fail_after(nth))
        try:
            model.forward_host(ids)
        except gpu.RuntimeFailure as exc:
            failures += 1
            assert exc.status == gpu.CUDA_ERROR and "injected" in str(exc)
        finally:
            gpu.check(lib.bfb_pool_fail_after(0))
        # whatever the pass had taken from the pool before the failure went back to it
        assert pool_stats(gpu)[1] == live_before, (nth, pool_stats(gpu), live_before)
        assert np.array_equal(model.forward_host(ids), want)
    assert failures >= 1, "no acquisition of the pass was hit by the injected failure"
    # the plain entry point too
    gpu.check(lib.bfb_pool_fail_after(1))
    p = C.c_void_p()
    assert lib.bfb_pool_acquire(1024, C.byref(p)) == gpu.CUDA_ERROR
    gpu.check(lib.bfb_pool_acquire(1024, C.byref(p)))
    gpu.check(lib.bfb_pool_release(p, 1024))
