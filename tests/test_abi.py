"""CPU-side checks of the C-ABI library: it loads, exports exactly what include/bfb200.h declares,
rejects bad arguments without touching a device, and its host logic (model structure, seeded inputs)
agrees with the reference. No compute entry point is exercised here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import bf_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "bfb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bfb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(bfb):
    declared = header_functions()
    assert declared, "no declarations parsed from include/bfb200.h"
    assert sorted(bfb.SIGNATURES) == declared


def test_library_exports_every_declared_symbol(bfb):
    handle = bfb.lib()
    for name in header_functions():
        assert getattr(handle, name) is not None
    assert bfb.lib().bfb_version() >= 100


def test_model_structure_matches_reference_layout(bfb):
    ops = O.lm_ops(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32)
    m = bfb.Model(ops)
    names = m.param_names()
    layout = O.param_layout(ops)
    assert names == [n for n, _ in layout]
    assert [m.param_shape(i) for i in range(len(names))] == [tuple(s) for _, s in layout]


def test_model_create_rejects_bad_pipelines(bfb):
    with pytest.raises(bfb.InvalidArgument):
        bfb.Model([{"kind": "embedding", "vocab": 8, "emb_dim": 6}, {"kind": "attention", "heads": 4}])
    with pytest.raises(bfb.InvalidArgument):
        bfb.Model([{"kind": "linear", "linear_out": 4}], input_last_dim=0)   # symbolic feature width
    with pytest.raises(bfb.InvalidArgument):
        bfb.Model([{"kind": "embedding", "vocab": 8, "emb_dim": 8}, {"kind": "bidirectional_attention", "heads": 2}])
    with pytest.raises(bfb.InvalidArgument):
        bfb.Model([])


def test_tensor_parallel_shapes_are_validated(bfb):
    ops = O.lm_ops(vocab=64, dim=32, layers=1, heads=4, hidden=48, max_seq=8)
    m = bfb.Model(ops, random_init=False)
    with pytest.raises(bfb.InvalidArgument):
        m.set_tensor_parallel(0, 3)      # 4 heads do not divide by 3
    with pytest.raises(bfb.InvalidArgument):
        m.set_tensor_parallel(2, 2)
    m.set_tensor_parallel(1, 2)
    assert m.param_names() == [n for n, _ in O.param_layout(ops)]


def test_synthetic_input_matches_reference(bfb, golden_c1_default):
    ops = O.lm_ops(vocab=256, dim=64, layers=2, heads=4, hidden=256, max_seq=32)
    ids = bfb.synthetic_input(ops, [-1, 32], batch=4, seed=42)
    assert np.array_equal(ids, golden_c1_default["ids"])


def test_argument_errors_need_no_device(bfb):
    lib = bfb.lib()
    st = lib.bfb_gemm(None, None, None, -1, 4, 4, bfb.F32, bfb.B_KN, bfb.F32, 0, None, None, 1.0, None, 0, None, None)
    assert st == bfb.INVALID_ARGUMENT and b"negative" in lib.bfb_last_error()
    st = lib.bfb_attention_fwd(None, None, None, None, None, None, bfb.F32, 1, 4, 4, 0, 16, 16, 16, 16, 16, 1.0, 0, 1,
                               None, None)
    assert st == bfb.INVALID_ARGUMENT
    st = lib.bfb_rmsnorm(None, 7, None, 0, 4, 4, 1e-6, None)
    assert st == bfb.INVALID_ARGUMENT
    st = lib.bfb_elementwise(99, None, None, None, None, 4, 0, None)
    assert st == bfb.INVALID_ARGUMENT
    # empty problems succeed without touching anything
    assert lib.bfb_gemm(None, None, None, 0, 4, 4, bfb.F32, bfb.B_KN, bfb.F32, 0, None, None, 1.0, None, 0, None, None) == 0
    assert lib.bfb_pool_release(None, 0) == 0


def test_no_cpu_fallback_without_device(bfb):
    if bfb.has_gpu():
        pytest.skip("a device is present")
    p = C.c_void_p()
    assert bfb.lib().bfb_pool_acquire(1024, C.byref(p)) == bfb.CUDA_ERROR
    ops = O.lm_ops(vocab=16, dim=8, layers=1, heads=2, hidden=16, max_seq=4)
    m = bfb.Model(ops)
    with pytest.raises(bfb.RuntimeFailure):
        m.forward_host(np.zeros((1, 4), dtype=np.float32))
    with pytest.raises(bfb.RuntimeFailure):
        m.set_param(0, np.zeros((16, 8), dtype=np.float32))


def test_bf16_bit_helpers_round_to_nearest_even(bfb):
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.4e38, 1e-40], dtype=np.float32)
    back = bfb.bf16_bits_to_f32(bfb.f32_to_bf16_bits(x))
    assert np.array_equal(back, O.round_bf16(x))


@pytest.mark.parametrize("count,threads,offset", [(0, 1, 0), (1, 1, 0), (7, 3, 0), (64, 1, 1), (100003, 4, 3), (4096, 16, 0)])
def test_host_widening_is_exact(count, threads, offset):
    """The host half of the bf16 result path runs without a device: every bf16 pattern, finite or not, must come out
    as the fp32 word with the same upper 16 bits, whatever the alignment of the destination and the thread split."""
    import blackforge_b200 as bfb
    rng = np.random.default_rng(count + threads)
    src = rng.integers(0, 1 << 16, size=count, dtype=np.uint16)
    if count >= 4:
        src[:4] = [0x7F80, 0xFF80, 0x7FC1, 0x8000]       # +inf, -inf, a NaN, -0
    backing = np.zeros(count + offset + 1, dtype=np.float32)
    dst = backing[offset:offset + count]
    rc = bfb.lib().bfb_host_widen_bf16(src.ctypes.data if count else None, dst.ctypes.data if count else None, count, threads)
    assert rc == bfb.OK
    assert np.array_equal(dst.view(np.uint32), src.astype(np.uint32) << 16)
    assert backing[:offset].tolist() == [0.0] * offset and backing[-1] == 0.0
    assert bfb.lib().bfb_host_widen_bf16(src.ctypes.data, dst.ctypes.data, count, 0) == bfb.INVALID_ARGUMENT


def test_checkpoint_index_reads_headers_only(bfb, tmp_path):
    """The header pass of the streaming loader (no device): names, shapes and data offsets of a file written in the
    reference's format, and the whole file's extent checked before anything would be loaded."""
    rng = np.random.default_rng(5)
    tensors = [("embedding1.table", rng.standard_normal((8, 6)).astype(np.float32)),
               ("feedforward4.b1", rng.standard_normal(16).astype(np.float32)),
               ("empty", np.zeros((0, 4), np.float32)),
               ("linear5.weight", rng.standard_normal((6, 8)).astype(np.float32))]
    path = str(tmp_path / "x.bfckpt")
    O.save_checkpoint(path, tensors)
    raw = open(path, "rb").read()
    index = bfb.checkpoint_index(path)
    assert [(n, s) for n, s, _, _ in index] == [(n, a.shape) for n, a in tensors]
    for (name, shape, offset, size), (_, want) in zip(index, tensors):
        assert size == want.nbytes
        assert np.array_equal(np.frombuffer(raw[offset:offset + size], np.float32).reshape(shape), want)
    for label, blob in (("magic", b"XXXXXXXX" + raw[8:]), ("cut_data", raw[:-3]), ("cut_header", raw[:14]),
                        ("cut_mid", raw[:index[1][2] + 2])):
        bad = str(tmp_path / label)
        open(bad, "wb").write(blob)
        with pytest.raises(bfb.RuntimeFailure) as e:
            bfb.checkpoint_index(bad)
        assert e.value.status == bfb.IO_ERROR, label
    with pytest.raises(bfb.RuntimeFailure) as e:
        bfb.checkpoint_index(str(tmp_path / "missing"))
    assert e.value.status == bfb.IO_ERROR
