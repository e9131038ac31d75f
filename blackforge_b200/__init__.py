"""blackforge_b200 — ctypes binding of libbfb200.so, the B200 backend for BlackForge's decoder-only
forward path (see include/bfb200.h for the C ABI and csrc/host/bfb200.hpp for the C++ operator API).

This package holds no compute of its own: every call goes through the C ABI into CUDA kernels. If the
library has not been built (python -m blackforge_b200.build) importing `lib()` fails loudly; there is
no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# BFB200_LIBRARY points at another build of the same library (e.g. an instrumented one) when set.
LIB_PATH = os.environ.get("BFB200_LIBRARY") or os.path.join(_HERE, "libbfb200.so")

OK, INVALID_ARGUMENT, CUDA_ERROR, TIMEOUT, UNSUPPORTED, IO_ERROR = range(6)
F32, BF16, FP8_E4M3 = 0, 1, 2
DT = {"fp8.e4m3": 0, "fp8.e5m2": 1, "fp16": 2, "bf16": 3, "tf32": 4, "fp32": 5}
OP_KINDS = ["linear", "silu", "relu", "gelu", "rmsnorm", "softmax", "embedding", "positional_embedding",
            "attention", "feedforward", "bidirectional_attention"]
EPI = {"none": 0, "bias": 1, "bias_silu": 2, "bias_residual": 3, "residual": 4}
B_KN, B_NK = 0, 1
EW = {"add": 0, "add_bias": 1, "add_bias_silu": 2, "add_bias_residual": 3, "silu": 4, "relu": 5, "gelu": 6}
ELEM_BYTES = {F32: 4, BF16: 2, FP8_E4M3: 1}


class BfbError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class InvalidArgument(BfbError, ValueError):
    """std::invalid_argument on the C++ side."""


class RuntimeFailure(BfbError, RuntimeError):
    """std::runtime_error on the C++ side (CUDA, I/O, timeout, unsupported)."""


class OpDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("input", C.c_int64), ("output", C.c_int64),
                ("linear_out_features", C.c_int64), ("embedding_vocab_size", C.c_int64),
                ("embedding_dim", C.c_int64), ("positional_max_seq_len", C.c_int64),
                ("attention_num_heads", C.c_int64), ("feedforward_hidden_dim", C.c_int64)]


class Precision(C.Structure):
    _fields_ = [("present", C.c_int32), ("storage", C.c_int32), ("compute", C.c_int32), ("accumulate", C.c_int32)]


_lib = None

# name -> (restype, argtypes); every symbol include/bfb200.h declares
_P, _I32, _I64, _F, _SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
SIGNATURES = {
    "bfb_last_error": (C.c_char_p, []),
    "bfb_version": (_I32, []),
    "bfb_device_count": (_I32, [C.POINTER(_I32)]),
    "bfb_set_device": (_I32, [_I32]),
    "bfb_pool_acquire": (_I32, [_SZ, C.POINTER(_P)]),
    "bfb_pool_release": (_I32, [_P, _SZ]),
    "bfb_pool_trim": (_I32, []),
    "bfb_pool_stats": (_I32, [C.POINTER(_SZ), C.POINTER(_SZ)]),
    "bfb_copy_h2d": (_I32, [_P, _P, _SZ, _P]),
    "bfb_copy_d2h": (_I32, [_P, _P, _SZ, _P]),
    "bfb_copy_d2d": (_I32, [_P, _P, _SZ, _P]),
    "bfb_memset_zero": (_I32, [_P, _SZ, _P]),
    "bfb_stream_synchronize": (_I32, [_P]),
    "bfb_embed_pos": (_I32, [_P, _P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _P, _P]),
    "bfb_add_positional": (_I32, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P]),
    "bfb_rmsnorm": (_I32, [_P, _I32, _P, _I32, _I64, _I64, _F, _P]),
    "bfb_softmax": (_I32, [_P, _P, _I64, _I64, _P]),
    "bfb_elementwise": (_I32, [_I32, _P, _P, _P, _P, _I64, _I64, _P]),
    "bfb_cast": (_I32, [_P, _I32, _P, _I32, _I64, _F, _P, _P]),
    "bfb_amax": (_I32, [_P, _I32, _I64, _P, _P]),
    "bfb_fp8_scale_from_amax": (_I32, [_P, _P, _P]),
    "bfb_rmsnorm_quantize_e4m3": (_I32, [_P, _I64, _I64, _F, _P, _P, _P, _P]),
    "bfb_rmsnorm_quantize_e4m3_from_stats": (_I32, [_P, _I64, _I64, _F, _P, _P, _P, _P, _P, _I32, _P]),
    "bfb_quantize_e4m3": (_I32, [_P, _I32, _I64, _P, _P, _P, _P]),
    "bfb_quantize_e4m3_static": (_I32, [_P, _I32, _I64, _P, _P, _P, _P]),
    "bfb_weight_prepare": (_I32, [_P, _P, _I32, _I64, _I64, _F, _P, _P]),
    "bfb_gemm": (_I32, [_P, _P, _P, _I64, _I64, _I64, _I32, _I32, _I32, _I32, _P, _P, _F, _P, _I32, _P, _P]),
    "bfb_row_sum_squares": (_I32, [_P, _I32, _P, _I64, _I64, _P]),
    "bfb_gemm_rmsnorm": (_I32, [_P, _P, _P, _I64, _I64, _I64, _I32, _I32, _I32, _P, _P, _P, _I32, _F, _P, _P, _P, _P]),
    "bfb_gemm_few_rows": (_I32, [_P, _P, _P, _I64, _I64, _I64, _I32, _I32, _I32, _P, _P, _F, _P, _I32, _F, _P, _P, _P]),
    "bfb_matmul_transpose_b": (_I32, [_P, _P, _P, _I64, _I64, _I64, _P]),
    "bfb_matmul_bf16_backward": (_I32, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "bfb_attention_fwd": (_I32, [_P, _P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64,
                                 _F, _I64, _I32, _P, _P]),
    "bfb_attention_fwd_maxima": (_I32, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _F, _I64,
                                        _P, _P]),
    "bfb_attention_bwd": (_I32, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64,
                                 _I64, _I64, _I64, _F, _I64, _I32, _P, _P]),
    "bfb_model_create": (_I32, [C.POINTER(OpDesc), _I32, _I64, C.c_uint32, C.POINTER(Precision), C.POINTER(_P)]),
    "bfb_model_create_uninitialised": (_I32, [C.POINTER(OpDesc), _I32, _I64, C.POINTER(Precision), C.POINTER(_P)]),
    "bfb_model_destroy": (None, [_P]),
    "bfb_model_set_tensor_parallel": (_I32, [_P, _I32, _I32]),
    "bfb_model_set_tensor_parallel_overlap": (_I32, [_P, _I32, _I32]),
    "bfb_set_shared_sm_mode": (_I32, [_I32, _I32]),
    "bfb_model_param_count": (_I32, [_P]),
    "bfb_model_param_name": (C.c_char_p, [_P, _I32]),
    "bfb_model_param_rank": (_I32, [_P, _I32]),
    "bfb_model_param_shape": (None, [_P, _I32, C.POINTER(_I64)]),
    "bfb_model_param_set": (_I32, [_P, _I32, _P]),
    "bfb_model_param_get": (_I32, [_P, _I32, _P]),
    "bfb_model_param_fill_normal": (_I32, [_P, _I32, C.c_uint64, _F]),
    "bfb_model_release_master_weights": (_I32, [_P]),
    "bfb_model_load_checkpoint": (_I32, [_P, C.c_char_p]),
    "bfb_model_save_checkpoint": (_I32, [_P, C.c_char_p]),
    "bfb_model_benchmark": (_I32, [_P, _P, C.POINTER(_I64), _I32, _I64, _I64, _P, _P, _I32, _P]),
    "bfb_model_load_checkpoint_streaming": (_I32, [_P, C.c_char_p, C.c_uint64, _P]),
    "bfb_model_load_checkpoint_cached": (_I32, [_P, C.c_char_p, C.c_uint64, _P]),
    "bfb_checkpoint_index": (_I32, [C.c_char_p, _I32, C.c_char_p, _I32, C.POINTER(_I32), C.POINTER(_I64),
                                    C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(_I32)]),
    "bfb_model_forward_incremental": (_I32, [_P, _P, C.POINTER(_I64), _I32, _I32, C.POINTER(_P), C.POINTER(_I64),
                                              C.POINTER(_I32), _P]),
    "bfb_model_reset_generation": (_I32, [_P]),
    "bfb_model_generation_position": (_I32, [_P, C.POINTER(_I64)]),
    "bfb_model_forward": (_I32, [_P, _P, C.POINTER(_I64), _I32, _I32, C.POINTER(_P), C.POINTER(_I64),
                                 C.POINTER(_I32), _P]),
    "bfb_model_forward_host": (_I32, [_P, _P, C.POINTER(_I64), _I32, _P, C.POINTER(_I64), C.POINTER(_I32)]),
    "bfb_model_forward_host_bf16": (_I32, [_P, _P, C.POINTER(_I64), _I32, _P, C.POINTER(_I64), C.POINTER(_I32)]),
    "bfb_host_transfer_bytes": (_I32, [C.POINTER(_I64), C.POINTER(_I64)]),
    "bfb_host_widen_bf16": (_I32, [_P, _P, _I64, _I32]),
    "bfb_launch_count": (_I64, [_I32]),
    "bfb_profile_enable": (_I32, [_I32]),
    "bfb_profile_reset": (_I32, []),
    "bfb_profile_read": (_I32, [_I32, C.POINTER(C.c_double), C.POINTER(_I64), C.POINTER(C.c_double)]),
    "bfb_synthetic_input": (_I32, [C.POINTER(OpDesc), _I32, C.POINTER(_I64), _I32, _I64, C.c_uint32, _P]),
    "bfb_selftest_bounded_wait": (_I32, [C.c_uint64, C.POINTER(_I32), _P]),
    "bfb_pool_fail_after": (_I32, [_I64]),
    "bfb_selftest_collective_watchdog": (_I32, [_I32, _I32, _I64, C.POINTER(_I32), C.POINTER(_I32)]),
    "bfb_tp_unique_id": (_I32, [_P]),
    "bfb_tp_init": (_I32, [_P, _I32, _I32]),
    "bfb_tp_allreduce_sum": (_I32, [_P, _I64, _I32, _P]),
    "bfb_gradients_average": (_I32, [_P, _P, _I32, _P]),
    "bfb_tp_destroy": (_I32, []),
}


def lib():
    """The loaded C-ABI library. Raises if it has not been built: there is no other implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m blackforge_b200.build` "
                               "(needs nvcc); blackforge_b200 has no CPU fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int):
    if status != OK:
        msg = lib().bfb_last_error().decode("utf-8", "replace")
        raise (InvalidArgument if status == INVALID_ARGUMENT else RuntimeFailure)(status, msg)


def has_gpu() -> bool:
    n = _I32(0)
    return lib().bfb_device_count(C.byref(n)) == OK and n.value > 0


# ---- bf16 / e4m3 helpers on the host (bit-level, for moving test data in and out) --------------------

def f32_to_bf16_bits(a) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- device buffers -------------------------------------------------------------------------------------

class DeviceBuffer:
    """A buffer from the library's device pool."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = _P()
        check(lib().bfb_pool_acquire(self.nbytes, C.byref(p)))
        self.ptr = p.value or 0

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        if a.nbytes:
            check(lib().bfb_copy_h2d(buf.ptr, a.ctypes.data, a.nbytes, None))
        return buf

    @classmethod
    def zeros(cls, nbytes: int) -> "DeviceBuffer":
        buf = cls(nbytes)
        if nbytes:
            check(lib().bfb_memset_zero(buf.ptr, nbytes, None))
        return buf

    def to_numpy(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            check(lib().bfb_copy_d2h(out.ctypes.data, self.ptr, out.nbytes, None))
        return out

    def free(self):
        if self.ptr:
            lib().bfb_pool_release(self.ptr, self.nbytes)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def upload(a, dtype: int) -> DeviceBuffer:
    """fp32 host data -> device buffer in `dtype` (conversion done on the device by bfb_cast)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    src = DeviceBuffer.from_numpy(a)
    if dtype == F32:
        return src
    dst = DeviceBuffer(a.size * ELEM_BYTES[dtype])
    check(lib().bfb_cast(src.ptr, F32, dst.ptr, dtype, a.size, 1.0, None, None))
    sync()
    src.free()
    return dst


def download(buf: DeviceBuffer, dtype: int, shape) -> np.ndarray:
    """Device buffer in `dtype` -> fp32 host array."""
    n = int(np.prod(shape)) if len(shape) else 1
    if dtype == F32:
        return buf.to_numpy(np.float32, shape)
    tmp = DeviceBuffer(n * 4)
    check(lib().bfb_cast(buf.ptr, dtype, tmp.ptr, F32, n, 1.0, None, None))
    out = tmp.to_numpy(np.float32, shape)
    tmp.free()
    return out


def sync(stream=None):
    check(lib().bfb_stream_synchronize(stream))


# ---- model ------------------------------------------------------------------------------------------------

def make_op_descs(ops: Sequence[dict]):
    arr = (OpDesc * len(ops))()
    for i, op in enumerate(ops):
        arr[i].kind = OP_KINDS.index(op["kind"])
        arr[i].input = op.get("input", i)
        arr[i].output = op.get("output", i + 1)
        arr[i].linear_out_features = op.get("linear_out", 0)
        arr[i].embedding_vocab_size = op.get("vocab", 0)
        arr[i].embedding_dim = op.get("emb_dim", 0)
        arr[i].positional_max_seq_len = op.get("max_seq", 0)
        arr[i].attention_num_heads = op.get("heads", 0)
        arr[i].feedforward_hidden_dim = op.get("hidden", 0)
    return arr


def make_precision(precision: Optional[dict]) -> Precision:
    p = Precision()
    if precision:
        p.present = 1
        p.storage = DT[precision.get("storage", "fp32")]
        p.compute = DT[precision.get("compute", "fp32")]
        p.accumulate = DT[precision.get("accumulate", "fp32")]
    return p


class Model:
    """bfb_model behind the C ABI (the device counterpart of blackforge::backend::cuda::Model)."""

    def __init__(self, ops: Sequence[dict], input_last_dim: int = 0, seed: int = 42,
                 precision: Optional[dict] = None, random_init: bool = True):
        self._ops = make_op_descs(ops)
        self._prec = make_precision(precision)
        self._h = _P()
        if random_init:
            check(lib().bfb_model_create(self._ops, len(ops), input_last_dim, seed, C.byref(self._prec), C.byref(self._h)))
        else:
            check(lib().bfb_model_create_uninitialised(self._ops, len(ops), input_last_dim, C.byref(self._prec),
                                                       C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().bfb_model_destroy(self._h)
            self._h = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_tensor_parallel(self, rank: int, world: int):
        check(lib().bfb_model_set_tensor_parallel(self._h, rank, world))

    def set_tensor_parallel_overlap(self, groups: int, reserved_sms: int):
        check(lib().bfb_model_set_tensor_parallel_overlap(self._h, groups, reserved_sms))

    def param_names(self) -> List[str]:
        return [lib().bfb_model_param_name(self._h, i).decode() for i in range(lib().bfb_model_param_count(self._h))]

    def param_shape(self, index: int) -> tuple:
        rank = lib().bfb_model_param_rank(self._h, index)
        s = (_I64 * max(rank, 1))()
        lib().bfb_model_param_shape(self._h, index, s)
        return tuple(s[i] for i in range(rank))

    def set_param(self, index: int, value):
        v = np.ascontiguousarray(value, dtype=np.float32)
        assert v.shape == self.param_shape(index), (v.shape, self.param_shape(index))
        check(lib().bfb_model_param_set(self._h, index, v.ctypes.data))

    def get_param(self, index: int) -> np.ndarray:
        out = np.empty(self.param_shape(index), dtype=np.float32)
        check(lib().bfb_model_param_get(self._h, index, out.ctypes.data))
        return out

    def fill_param_normal(self, index: int, seed: int, sigma: float):
        check(lib().bfb_model_param_fill_normal(self._h, index, seed, sigma))

    def release_master_weights(self):
        check(lib().bfb_model_release_master_weights(self._h))

    def set_params(self, params: Dict[str, np.ndarray]):
        for i, name in enumerate(self.param_names()):
            if name in params:
                self.set_param(i, params[name])

    def load_checkpoint(self, path: str):
        check(lib().bfb_model_load_checkpoint(self._h, path.encode()))

    def load_checkpoint_streaming(self, path: str, chunk_bytes: int = 0) -> dict:
        """load_checkpoint with its figures: tensors, file / read / uploaded bytes, seconds."""
        stats = CheckpointLoadStats()
        check(lib().bfb_model_load_checkpoint_streaming(self._h, path.encode(), chunk_bytes, C.byref(stats)))
        return {name: getattr(stats, name) for name, _ in CheckpointLoadStats._fields_}

    def load_checkpoint_cached(self, path: str, chunk_bytes: int = 0) -> dict:
        """Streaming load that keeps / uses a cache of the converted GEMM weights beside the file."""
        stats = CheckpointLoadStats()
        check(lib().bfb_model_load_checkpoint_cached(self._h, path.encode(), chunk_bytes, C.byref(stats)))
        return {name: getattr(stats, name) for name, _ in CheckpointLoadStats._fields_}

    def save_checkpoint(self, path: str):
        check(lib().bfb_model_save_checkpoint(self._h, path.encode()))

    def forward_host(self, x) -> np.ndarray:
        """Host ids in, host logits out (the `blackforge run` path)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        shape = (_I64 * x.ndim)(*x.shape)
        out_shape = (_I64 * 8)()
        out_rank = _I32(0)
        check(lib().bfb_model_forward_host(self._h, x.ctypes.data, shape, x.ndim, None, out_shape, C.byref(out_rank)))
        out = np.empty([out_shape[i] for i in range(out_rank.value)], dtype=np.float32)
        check(lib().bfb_model_forward_host(self._h, x.ctypes.data, shape, x.ndim, out.ctypes.data, out_shape,
                                           C.byref(out_rank)))
        return out

    def benchmark(self, x, warmup: int = 1, measured: int = 5) -> dict:
        """Device-timed passes over the host array `x` (uploaded once): mean ms, samples/s, the reference's memory
        estimate and the mean device time of every pipeline operation inside the pass."""
        a = np.ascontiguousarray(x, dtype=np.float32)
        d_in = DeviceBuffer.from_numpy(a)
        shape = (_I64 * a.ndim)(*a.shape)
        res = BenchmarkResult()
        count = max(1, len(self._ops))
        per_op = (OpBenchmark * count)()
        check(lib().bfb_model_benchmark(self._h, d_in.ptr, shape, a.ndim, warmup, measured, C.byref(res), per_op, count, None))
        return {"mean_ms": res.mean_ms, "samples_per_second": res.samples_per_second,
                "estimated_memory_bytes": res.estimated_memory_bytes, "warmup": res.warmup_iterations,
                "measured": res.measured_iterations,
                "per_operation": [(per_op[i].name.decode(), per_op[i].index, per_op[i].mean_ms)
                                  for i in range(min(count, res.op_count))]}

    def forward_host_bf16(self, x) -> np.ndarray:
        """Host ids in, host logits out as bf16 bit patterns (uint16); needs storage bf16."""
        a = np.ascontiguousarray(x, dtype=np.float32)
        s = (_I64 * a.ndim)(*a.shape)
        out_shape = (_I64 * 8)()
        out_rank = _I32(0)
        check(lib().bfb_model_forward_host_bf16(self._h, a.ctypes.data, s, a.ndim, None, out_shape, C.byref(out_rank)))
        oshape = tuple(out_shape[i] for i in range(out_rank.value))
        out = np.empty(oshape, dtype=np.uint16)
        check(lib().bfb_model_forward_host_bf16(self._h, a.ctypes.data, s, a.ndim, out.ctypes.data, out_shape,
                                                C.byref(out_rank)))
        return out

    def forward_device(self, d_input: int, shape: Sequence[int], trusted: bool = False, stream=None):
        """Device ids in, device logits out: returns (DeviceBuffer, shape). No synchronisation."""
        s = (_I64 * len(shape))(*shape)
        out_shape = (_I64 * 8)()
        out_rank = _I32(0)
        out_ptr = _P()
        check(lib().bfb_model_forward(self._h, d_input, s, len(shape), int(trusted), C.byref(out_ptr), out_shape,
                                      C.byref(out_rank), stream))
        oshape = tuple(out_shape[i] for i in range(out_rank.value))
        buf = DeviceBuffer.__new__(DeviceBuffer)
        buf.ptr = out_ptr.value or 0
        buf.nbytes = int(np.prod(oshape)) * 4
        return buf, oshape

    def forward_incremental_device(self, d_new_ids: int, shape: Sequence[int], trusted: bool = False, stream=None):
        """Generation: device ids of the NEW positions in, their device logits out: (DeviceBuffer, shape)."""
        s = (_I64 * len(shape))(*shape)
        out_shape = (_I64 * 8)()
        out_rank = _I32(0)
        out_ptr = _P()
        check(lib().bfb_model_forward_incremental(self._h, d_new_ids, s, len(shape), int(trusted), C.byref(out_ptr),
                                                  out_shape, C.byref(out_rank), stream))
        oshape = tuple(out_shape[i] for i in range(out_rank.value))
        buf = DeviceBuffer.__new__(DeviceBuffer)
        buf.ptr = out_ptr.value or 0
        buf.nbytes = int(np.prod(oshape)) * 4
        return buf, oshape

    def forward_incremental(self, new_ids) -> np.ndarray:
        """Host convenience: ids of the new positions [batch, new_len] in, their logits out."""
        a = np.ascontiguousarray(new_ids, dtype=np.float32)
        d = DeviceBuffer.from_numpy(a)
        out, shape = self.forward_incremental_device(d.ptr, a.shape)
        res = out.to_numpy(np.float32, shape)
        out.free()
        d.free()
        return res

    def reset_generation(self):
        check(lib().bfb_model_reset_generation(self._h))

    def generation_position(self) -> int:
        pos = _I64(0)
        check(lib().bfb_model_generation_position(self._h, C.byref(pos)))
        return int(pos.value)


def host_transfer_bytes():
    """(host-to-device, device-to-host) bytes of this thread's latest Model.forward_host."""
    a, b = _I64(0), _I64(0)
    check(lib().bfb_host_transfer_bytes(C.byref(a), C.byref(b)))
    return int(a.value), int(b.value)


def synthetic_input(ops: Sequence[dict], input_shape: Sequence[int], batch: int, seed: int = 42) -> np.ndarray:
    """Executor::makeSyntheticInput: -1 in input_shape marks the symbolic batch dimension."""
    descs = make_op_descs(ops)
    shape = (_I64 * len(input_shape))(*input_shape)
    dims = [batch if d < 0 else d for d in input_shape]
    out = np.empty(dims, dtype=np.float32)
    check(lib().bfb_synthetic_input(descs, len(ops), shape, len(input_shape), batch, seed, out.ctypes.data))
    return out


# ---- tensor-parallel communicator ---------------------------------------------------------------------------

def tp_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    check(lib().bfb_tp_unique_id(buf))
    return buf.raw


class OpBenchmark(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("index", C.c_int32), ("mean_ms", C.c_double)]


class BenchmarkResult(C.Structure):
    _fields_ = [("warmup_iterations", C.c_int64), ("measured_iterations", C.c_int64), ("mean_ms", C.c_double),
                ("samples_per_second", C.c_double), ("estimated_memory_bytes", C.c_uint64), ("op_count", C.c_int32)]


class CheckpointLoadStats(C.Structure):
    _fields_ = [("tensors", C.c_int64), ("file_bytes", C.c_uint64), ("read_bytes", C.c_uint64),
                ("uploaded_bytes", C.c_uint64), ("seconds", C.c_double), ("cache_hit", C.c_int32),
                ("cache_bytes", C.c_uint64)]


def checkpoint_index(path: str) -> list:
    """Header pass over a BFCKPT1 file (no device): [(name, shape, data_offset, data_bytes), ...]."""
    count = C.c_int32(0)
    check(lib().bfb_checkpoint_index(path.encode(), -1, None, 0, None, None, None, None, C.byref(count)))
    out = []
    for i in range(count.value):
        name = C.create_string_buffer(1024)
        rank, dims = C.c_int32(0), (C.c_int64 * 8)()
        off, size = C.c_uint64(0), C.c_uint64(0)
        check(lib().bfb_checkpoint_index(path.encode(), i, name, 1024, C.byref(rank), dims, C.byref(off), C.byref(size), None))
        out.append((name.value.decode(), tuple(dims[d] for d in range(rank.value)), off.value, size.value))
    return out


def set_shared_sm_mode(dynamic_tiles: bool, reserved_sms: int = 0):
    check(lib().bfb_set_shared_sm_mode(1 if dynamic_tiles else 0, reserved_sms))


def tp_init(unique_id: bytes, rank: int, world: int):
    assert len(unique_id) == 128
    check(lib().bfb_tp_init(C.create_string_buffer(unique_id, 128), rank, world))


def tp_destroy():
    check(lib().bfb_tp_destroy())
