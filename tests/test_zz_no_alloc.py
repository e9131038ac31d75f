"""bfb_quantize_e4m3_static — the entry point for hosts that cannot allocate device memory at call time
(an engine that owns the whole GPU arena, a serving loop that must stay out of the device allocator).
It has to give exactly what bfb_quantize_e4m3 gives, call after call, while keeping its scratch in the
library's fixed array. Collected last on purpose: a failure here cannot hide another test's result."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def quantize(gpu, fn, x, dtype, weight_inverse):
    src = gpu.upload(x, dtype)
    out = gpu.DeviceBuffer(x.size)
    scales = gpu.DeviceBuffer.zeros(12)
    winv = gpu.DeviceBuffer.from_numpy(np.array([weight_inverse], np.float32))
    gpu.check(fn(src.ptr, dtype, x.size, out.ptr, scales.ptr, winv.ptr, None))
    gpu.sync()
    return out.to_numpy(np.uint8, (x.size,)), scales.to_numpy(np.float32, (3,))


def test_static_scratch_variant_matches_pool_variant_twice_in_a_row(gpu):
    lib = gpu.lib()
    rng = np.random.default_rng(2024)
    # second call is smaller and has a smaller maximum: stale partial maxima from the first must not leak in
    cases = [((rng.standard_normal(8192 * 40 + 123) * 5).astype(np.float32), gpu.BF16, 0.5),
             ((rng.standard_normal(8192 * 3 + 7) * 0.01).astype(np.float32), gpu.F32, 2.0)]
    for x, dtype, winv in cases:
        want_q, want_s = quantize(gpu, lib.bfb_quantize_e4m3, x, dtype, winv)
        got_q, got_s = quantize(gpu, lib.bfb_quantize_e4m3_static, x, dtype, winv)
        # integer / bit-level work: exact equality, as everywhere else in the e4m3 tests
        assert np.array_equal(got_s, want_s)
        assert np.array_equal(got_q, want_q)


def test_static_scratch_variant_takes_no_device_memory(gpu):
    """The property the entry point exists for: after one warm-up call (address lookup, module load) a call takes
    nothing from the library's device pool and leaves the device's free memory where it was. The pool variant,
    measured the same way, does take its scratch from the pool."""
    import ctypes as C
    import torch

    lib = gpu.lib()
    x = (np.random.default_rng(7).standard_normal(8192 * 64) * 3).astype(np.float32)
    src = gpu.upload(x, gpu.BF16)
    out = gpu.DeviceBuffer(x.size)
    scales = gpu.DeviceBuffer.zeros(12)

    def pool():
        cached, live = C.c_size_t(0), C.c_size_t(0)
        gpu.check(lib.bfb_pool_stats(C.byref(cached), C.byref(live)))
        return cached.value, live.value

    gpu.check(lib.bfb_quantize_e4m3_static(src.ptr, gpu.BF16, x.size, out.ptr, scales.ptr, None, None))   # warm-up
    gpu.sync()
    gpu.check(lib.bfb_pool_trim())          # nothing cached: an acquisition would have to show up as new memory
    before_pool, before_free = pool(), torch.cuda.mem_get_info()[0]
    gpu.check(lib.bfb_quantize_e4m3_static(src.ptr, gpu.BF16, x.size, out.ptr, scales.ptr, None, None))
    gpu.sync()
    assert pool() == before_pool
    assert torch.cuda.mem_get_info()[0] == before_free
    # the same measurement sees the pool variant's scratch (kept cached by the pool after the call)
    gpu.check(lib.bfb_quantize_e4m3(src.ptr, gpu.BF16, x.size, out.ptr, scales.ptr, None, None))
    gpu.sync()
    assert pool()[0] > before_pool[0]


def test_static_scratch_variant_refuses_oversized_tensors(gpu):
    lib = gpu.lib()
    tiny = gpu.DeviceBuffer.zeros(64)
    too_many = 65536 * 8192 + 1
    st = lib.bfb_quantize_e4m3_static(tiny.ptr, gpu.BF16, too_many, tiny.ptr, tiny.ptr, None, None)
    assert st == gpu.INVALID_ARGUMENT and b"536870912" in lib.bfb_last_error()
    # the largest accepted count is not rejected by the size check (empty input: nothing is read)
    assert lib.bfb_quantize_e4m3_static(None, gpu.BF16, 0, None, tiny.ptr, None, None) == gpu.OK
