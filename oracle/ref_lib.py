"""TEST INFRASTRUCTURE — ctypes access to oracle/_ref/libbf_ref.so.

The library is the reference's own CPU backend (blackforge::backend::cpu) and front end, compiled
unmodified by oracle/Makefile; this module only marshals numpy arrays in and out of it. It is used
by the tests (to validate the numpy restatement in oracle/bf_oracle.py and as the parity checker),
by the golden-fixture generator and by the benchmark's CPU-baseline leg. Product code never
imports it.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libbf_ref.so")

# dtype codes shared with ref_shim.cpp (order of sema::DType)
DTYPE_CODES = {"fp8.e4m3": 0, "fp8.e5m2": 1, "fp16": 2, "bf16": 3, "tf32": 4, "fp32": 5}

# ir::OpKind enumerators in declaration order (include/blackforge/ir/operation.hpp:11-12)
OP_KINDS = ["linear", "silu", "relu", "gelu", "rmsnorm", "softmax", "embedding",
            "positional_embedding", "attention", "feedforward", "bidirectional_attention"]


class RefError(Exception):
    """Raised when the reference threw; .kind is 'invalid_argument' or 'runtime_error'."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.kind = "invalid_argument" if code == 1 else "runtime_error"


_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise FileNotFoundError(f"{LIB_PATH} missing: run `make -C oracle` where the reference sources exist")
        _lib = C.CDLL(LIB_PATH)
        _lib.refLastError.restype = C.c_char_p
        _lib.refResultCount.restype = C.c_int64
        _lib.refModelParamName.restype = C.c_char_p
        _lib.refSeedFor.restype = C.c_uint
        _lib.refSeedFor.argtypes = [C.c_uint, C.c_uint64, C.c_uint]
    return _lib


def _check(code: int):
    if code != 0:
        raise RefError(code, lib().refLastError().decode("utf-8", "replace"))


def _t(a) -> tuple:
    a = np.ascontiguousarray(a, dtype=np.float32)
    shape = (C.c_int64 * max(a.ndim, 1))(*a.shape)
    return a, (a.ctypes.data_as(C.c_void_p), shape, C.c_int(a.ndim))


def _result() -> np.ndarray:
    l = lib()
    rank = l.refResultRank()
    shape = (C.c_int64 * max(rank, 1))()
    l.refResultShape(shape)
    out = np.empty([shape[i] for i in range(rank)], dtype=np.float32)
    if out.size:
        l.refResultCopy(out.ctypes.data_as(C.c_void_p))
    return out


def _call(fn, *tensors, extra: Sequence = ()):
    keep, args = [], []
    for t in tensors:
        a, packed = _t(t)
        keep.append(a)
        args.extend(packed)
    _check(fn(*args, *extra))
    return _result()


# ---- operators -------------------------------------------------------------------------------

def silu(x): return _call(lambda *a: lib().refOpUnary(0, *a), x)
def relu(x): return _call(lambda *a: lib().refOpUnary(1, *a), x)
def gelu(x): return _call(lambda *a: lib().refOpUnary(2, *a), x)
def rmsnorm(x): return _call(lambda *a: lib().refOpUnary(3, *a), x)
def softmax(x): return _call(lambda *a: lib().refOpUnary(4, *a), x)


def _binary(which, a, b, extra=0):
    return _call(lambda *args: lib().refOpBinary(which, *args), a, b, extra=(C.c_int64(extra),))


def add(a, b): return _binary(0, a, b)
def add_bias(x, bias): return _binary(1, x, bias)
def matmul(a, b): return _binary(2, a, b)
def matmul_transpose_b(a, b): return _binary(3, a, b)
def embedding_lookup(ids, table): return _binary(4, ids, table)
def add_positional_embedding(x, table): return _binary(5, x, table)
def add_positional_embedding_at(x, table, offset): return _binary(6, x, table, offset)


def linear(x, w, b): return _call(lib().refOpLinear, x, w, b)
def feed_forward(x, w1, b1, w2, b2): return _call(lib().refOpFeedForward, x, w1, b1, w2, b2)


def self_attention(x, wq, wk, wv, wo, num_heads):
    return _call(lib().refOpSelfAttention, x, wq, wk, wv, wo, extra=(C.c_int64(num_heads),))


def quantize(x, dtype: str):
    return _call(lib().refOpQuantize, x, extra=(C.c_int(DTYPE_CODES[dtype]),))


def random_tensor(shape, seed: int):
    s = (C.c_int64 * len(shape))(*shape)
    _check(lib().refRandomTensor(s, len(shape), C.c_uint(seed)))
    return _result()


def seed_for(base: int, value_id: int, salt: int) -> int:
    return lib().refSeedFor(base, value_id, salt)


# ---- front end + Executor + Model -----------------------------------------------------------

class Compiled:
    """A .bf program run through the reference's Lexer/Parser/SemanticAnalyzer/IRBuilder."""

    def __init__(self, source: str):
        self._h = C.c_void_p()
        _check(lib().refCompile(source.encode(), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.refCompiledFree(self._h)
            self._h = None

    def precision(self) -> Optional[dict]:
        s, c, a = C.c_int(), C.c_int(), C.c_int()
        if not lib().refCompiledPrecision(self._h, C.byref(s), C.byref(c), C.byref(a)):
            return None
        names = {v: k for k, v in DTYPE_CODES.items()}
        return {"storage": names[s.value], "compute": names[c.value], "accumulate": names[a.value]}

    def ops(self) -> list:
        """The pipeline as a list of dicts mirroring ir::Operation."""
        out = []
        for i in range(lib().refCompiledOpCount(self._h)):
            f = (C.c_int64 * 9)()
            lib().refCompiledOp(self._h, i, f)
            out.append({"kind": OP_KINDS[f[0]], "input": f[1], "output": f[2], "linear_out": f[3],
                        "vocab": f[4], "emb_dim": f[5], "max_seq": f[6], "heads": f[7], "hidden": f[8]})
        return out

    def input_shape(self) -> list:
        rank = lib().refCompiledInputRank(self._h)
        s = (C.c_int64 * max(rank, 1))()
        lib().refCompiledInputShape(self._h, s)
        return [s[i] for i in range(rank)]

    def synthetic_input(self, seed: int, batch: int) -> np.ndarray:
        _check(lib().refExecutorSyntheticInput(self._h, C.c_uint(seed), C.c_int64(batch)))
        return _result()

    def executor_run(self, seed: int, x, use_precision: bool = False) -> np.ndarray:
        a, packed = _t(x)
        _check(lib().refExecutorRun(self._h, C.c_uint(seed), *packed, C.c_int(int(use_precision))))
        return _result()


class Model:
    """blackforge::backend::cpu::Model behind the shim."""

    def __init__(self, compiled: Compiled, seed: int = 42, precision=None):
        self._c = compiled
        self._m = C.c_void_p()
        if precision is None or precision is False:
            _check(lib().refModelNew(compiled._h, C.c_uint(seed), 0, C.byref(self._m)))
        elif precision is True:
            _check(lib().refModelNew(compiled._h, C.c_uint(seed), 1, C.byref(self._m)))
        else:
            _check(lib().refModelNewWithPrecision(
                compiled._h, C.c_uint(seed), DTYPE_CODES[precision["storage"]], DTYPE_CODES[precision["compute"]],
                DTYPE_CODES[precision.get("accumulate", "fp32")], C.byref(self._m)))

    def __del__(self):
        if getattr(self, "_m", None) and _lib is not None:
            _lib.refModelFree(self._m)
            self._m = None

    def forward(self, x) -> np.ndarray:
        a, packed = _t(x)
        _check(lib().refModelForward(self._m, *packed))
        return _result()

    def load_checkpoint(self, path: str):
        _check(lib().refModelLoadCheckpoint(self._m, path.encode()))

    def save_checkpoint(self, path: str):
        _check(lib().refModelSaveCheckpoint(self._m, path.encode()))

    def param_names(self) -> list:
        return [lib().refModelParamName(self._m, i).decode() for i in range(lib().refModelParamCount(self._m))]

    def param(self, index: int) -> np.ndarray:
        _check(lib().refModelParamFetch(self._m, index))
        return _result()

    def set_param(self, index: int, value):
        a, packed = _t(value)
        _check(lib().refModelParamSet(self._m, index, *packed))


# ---- the reference's CUDA backend (oracle/_ref/libbf_ref_cuda.so, `make -C oracle cuda`) ------------------------
# A second library that holds the reference's front end, CPU backend AND its unmodified CUDA backend (cuBLAS /
# cuBLASLt), so that the GPU parity tests can compare this repository's kernels with the reference's own device
# results. Programs are compiled through this library's own front end: handles do not cross libraries.

CUDA_LIB_PATH = os.path.join(_HERE, "_ref", "libbf_ref_cuda.so")
_cuda_lib = None


def cuda_available() -> bool:
    return os.path.exists(CUDA_LIB_PATH)


def cuda_lib():
    global _cuda_lib
    if _cuda_lib is None:
        if not cuda_available():
            raise FileNotFoundError(f"{CUDA_LIB_PATH} missing: run `make -C oracle cuda` where the reference sources exist")
        _cuda_lib = C.CDLL(CUDA_LIB_PATH)
        _cuda_lib.refLastError.restype = C.c_char_p
        _cuda_lib.refCudaLastError.restype = C.c_char_p
        _cuda_lib.refCudaResultCount.restype = C.c_int64
        _cuda_lib.refCudaModelParamName.restype = C.c_char_p
    return _cuda_lib


def _cuda_check(code: int, front_end: bool = False):
    if code != 0:
        l = cuda_lib()
        raise RefError(code, (l.refLastError() if front_end else l.refCudaLastError()).decode("utf-8", "replace"))


def _cuda_result() -> np.ndarray:
    l = cuda_lib()
    rank = l.refCudaResultRank()
    shape = (C.c_int64 * max(rank, 1))()
    l.refCudaResultShape(shape)
    out = np.empty([shape[i] for i in range(rank)], dtype=np.float32)
    if out.size:
        l.refCudaResultCopy(out.ctypes.data_as(C.c_void_p))
    return out


class CudaModel:
    """blackforge::backend::cuda::Model (the reference's own device path) built from program text."""

    def __init__(self, source: str, seed: int = 42, precision: Optional[dict] = None):
        l = cuda_lib()
        self._c = C.c_void_p()
        self._m = C.c_void_p()
        _cuda_check(l.refCompile(source.encode(), C.byref(self._c)), front_end=True)
        if precision is None:
            codes = (5, -1, 5)
        else:
            codes = (DTYPE_CODES[precision["storage"]], DTYPE_CODES[precision["compute"]],
                     DTYPE_CODES[precision.get("accumulate", "fp32")])
        _cuda_check(l.refCudaModelNew(self._c, C.c_uint(seed), *codes, C.byref(self._m)))

    def close(self):
        if getattr(self, "_m", None) and _cuda_lib is not None:
            _cuda_lib.refCudaModelFree(self._m)
            self._m = None
        if getattr(self, "_c", None) and _cuda_lib is not None:
            _cuda_lib.refCompiledFree(self._c)
            self._c = None

    def __del__(self):
        self.close()

    def param_names(self) -> list:
        l = cuda_lib()
        return [l.refCudaModelParamName(self._m, i).decode() for i in range(l.refCudaModelParamCount(self._m))]

    def set_param(self, index: int, value):
        a, packed = _t(value)
        _cuda_check(cuda_lib().refCudaModelParamSet(self._m, index, *packed))

    def forward(self, x) -> np.ndarray:
        a, packed = _t(x)
        _cuda_check(cuda_lib().refCudaModelForward(self._m, *packed))
        return _cuda_result()

    def forward_incremental(self, new_ids) -> np.ndarray:
        a, packed = _t(new_ids)
        _cuda_check(cuda_lib().refCudaModelForwardIncremental(self._m, *packed))
        return _cuda_result()

    def reset_generation(self):
        _cuda_check(cuda_lib().refCudaModelResetGeneration(self._m))

    def generation_timed(self, prompt, step_ids) -> float:
        """Device milliseconds per single-token step after the prompt (CUDA events)."""
        p = np.ascontiguousarray(prompt, dtype=np.float32)
        s = np.ascontiguousarray(step_ids, dtype=np.float32)
        ms = C.c_double(0.0)
        _cuda_check(cuda_lib().refCudaModelGenerationTimed(
            self._m, p.ctypes.data_as(C.c_void_p), C.c_int64(p.shape[0]), C.c_int64(p.shape[1]),
            s.ctypes.data_as(C.c_void_p), C.c_int64(s.shape[1]), C.byref(ms)))
        return ms.value

    def forward_timed(self, x, warmup: int = 1, iters: int = 3) -> float:
        """Device milliseconds per forward pass (CUDA events; input uploaded once, results left on the device)."""
        a, packed = _t(x)
        ms = C.c_double(0.0)
        _cuda_check(cuda_lib().refCudaModelForwardTimed(self._m, *packed, C.c_int(warmup), C.c_int(iters), C.byref(ms)))
        return ms.value


def cuda_fused_attention(q, k, v, num_heads: int, scale: float, old_len: int = 0) -> np.ndarray:
    """fusedAttentionForward of the reference on fp32 q [batch, newLen, dim], k / v [batch, totalLen, dim]."""
    qa, ka, va = (np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v))
    qs, ks = (C.c_int64 * 3)(*qa.shape), (C.c_int64 * 3)(*ka.shape)
    _cuda_check(cuda_lib().refCudaFusedAttention(qa.ctypes.data_as(C.c_void_p), qs, ka.ctypes.data_as(C.c_void_p), ks,
                                                 va.ctypes.data_as(C.c_void_p), C.c_int64(num_heads), C.c_float(scale),
                                                 C.c_int64(old_len)))
    return _cuda_result()


def cuda_fused_attention_timed(q, k, v, num_heads: int, scale: float, old_len: int = 0, iters: int = 3):
    """(output, device milliseconds per call) of the reference's fusedAttentionForward."""
    qa, ka, va = (np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v))
    qs, ks = (C.c_int64 * 3)(*qa.shape), (C.c_int64 * 3)(*ka.shape)
    ms = C.c_double(0.0)
    _cuda_check(cuda_lib().refCudaFusedAttentionTimed(
        qa.ctypes.data_as(C.c_void_p), qs, ka.ctypes.data_as(C.c_void_p), ks, va.ctypes.data_as(C.c_void_p),
        C.c_int64(num_heads), C.c_float(scale), C.c_int64(old_len), C.c_int(iters), C.byref(ms)))
    return _cuda_result(), ms.value


def cuda_fused_attention_backward(d_out, q, k, v, num_heads: int, scale: float, old_len: int = 0, iters: int = 0):
    """The reference's fusedAttentionForward + fusedAttentionBackward on fp32 operands: a dict with out, m, l, dq, dk,
    dv (and ms, the device time of one backward call, when iters > 0)."""
    ga, qa, ka, va = (np.ascontiguousarray(t, dtype=np.float32) for t in (d_out, q, k, v))
    qs, ks = (C.c_int64 * 3)(*qa.shape), (C.c_int64 * 3)(*ka.shape)
    batch, new_len, _ = qa.shape
    res = {"out": np.empty_like(qa), "m": np.empty((batch, num_heads, new_len), np.float32),
           "l": np.empty((batch, num_heads, new_len), np.float32), "dq": np.empty_like(qa), "dk": np.empty_like(ka),
           "dv": np.empty_like(ka)}
    ms = C.c_double(0.0)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    _cuda_check(cuda_lib().refCudaFusedAttentionBackward(
        ptr(ga), ptr(qa), qs, ptr(ka), ks, ptr(va), C.c_int64(num_heads), C.c_float(scale), C.c_int64(old_len),
        ptr(res["out"]), ptr(res["m"]), ptr(res["l"]), ptr(res["dq"]), ptr(res["dk"]), ptr(res["dv"]), C.c_int(iters),
        C.byref(ms)))
    if iters > 0:
        res["ms"] = ms.value
    return res


def cuda_matmul_bf16_backward(a, b, grad):
    """(dA, dB) of the reference's matmulBf16Backward (cuBLASLt, bf16 operands, fp32 results) for fp32 a [m,k], b [k,n],
    grad [m,n]."""
    aa, ba, ga = (np.ascontiguousarray(t, dtype=np.float32) for t in (a, b, grad))
    (m, k), n = aa.shape, ba.shape[1]
    d_a, d_b = np.empty((m, k), np.float32), np.empty((k, n), np.float32)
    ptr = lambda t: t.ctypes.data_as(C.c_void_p)
    _cuda_check(cuda_lib().refCudaMatmulBf16Backward(ptr(aa), ptr(ba), ptr(ga), C.c_int64(m), C.c_int64(k), C.c_int64(n),
                                                     ptr(d_a), ptr(d_b)))
    return d_a, d_b


def cuda_lt_gemm_timed(a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int, c_is_bf16: bool, warmup: int,
                       iters: int) -> float:
    """Device milliseconds per cublasLtMatmul call configured as the reference's bf16Gemm configures it, on the
    caller's device buffers: A [m, k] bf16, B [k, n] bf16, C [m, n] fp32 (the reference's) or bf16, all row-major."""
    ms = C.c_double(0.0)
    _cuda_check(cuda_lib().refCudaLtGemmTimed(C.c_void_p(a_ptr), C.c_void_p(b_ptr), C.c_void_p(c_ptr), C.c_int64(m),
                                              C.c_int64(n), C.c_int64(k), C.c_int(1 if c_is_bf16 else 0),
                                              C.c_int(warmup), C.c_int(iters), C.byref(ms)))
    return ms.value
