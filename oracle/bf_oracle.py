"""TEST INFRASTRUCTURE — numpy restatement of BlackForge's CPU forward path (the parity oracle).

This file is the checker the GPU parity tests compare against; it is never imported by the
product. Every function follows one reference function (path:line inside the reference project)
and keeps its arithmetic order where numpy allows it:

* matmul / matmulTransposeB accumulate in float32 one k at a time, the order of the reference's
  triple loops, so results are bit-identical to the reference built without FMA contraction;
* rmsnorm and softmax accumulate in float64 column by column, as the reference does;
* silu / gelu use float32 exp/tanh (numpy's may differ from glibc's by one ulp).

PINNING. The restatement is pinned two ways (tests/test_oracle.py): against the reference's own
known-answer tests re-expressed as inputs (2x2 matmul = 19/22/43/50, linear with identity weight,
unit-RMS rows, softmax rows summing to one, fp8 saturation at 448 and 57344, bf16 idempotence,
causal-mask invariance, zero-weight identity) and against outputs of the reference itself
(oracle/_ref, built from the reference sources) on seeded inputs, live when that library is
present and through the committed fixtures in tests/golden/ otherwise.

Two precision semantics are restated, because the reference has two:
* `cpu_policy`  — src/backend/cpu/model.cpp:174-239: `storage` rounds the input and every op
  output; `compute` rounds both matmul operands of `linear` ops ONLY.
* `cuda_policy` — src/backend/cuda/model.cu:139-140,275-300 with ops_tensorcore.cu:308-327: when
  compute == bf16 every GEMM (linear, Q/K/V/Out, both feed-forward GEMMs) rounds both operands to
  bf16 and accumulates in fp32; the attention core, norms, biases and residuals stay fp32.
The fp8 GEMM (per-tensor amax scales) has no reference implementation; `fp8_scaled_matmul` states
the arithmetic this project defines for it, built on the reference's e4m3 rounding rule —
"parity unpinned" for that one function.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

F32 = np.float32
RMS_EPS = F32(1e-6)            # src/backend/cpu/ops.cpp:14
GELU_COEFF = F32(0.044715)      # src/backend/cpu/ops.cpp:12
SQRT_2_OVER_PI = F32(0.7978845608)  # src/backend/cpu/ops.cpp:13


class InvalidArgument(ValueError):
    """Stands for std::invalid_argument thrown by the reference."""


class RuntimeFailure(RuntimeError):
    """Stands for std::runtime_error thrown by the reference."""


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=F32)


# ---- elementwise (src/backend/cpu/ops.cpp:113-158, 183-201) --------------------------------------

def add(a, b):
    a, b = _f32(a), _f32(b)
    if a.shape != b.shape:
        raise InvalidArgument("add: shape mismatch")
    return a + b


def scale(x, factor):
    return _f32(x) * F32(factor)


def add_bias(x, bias):
    x, bias = _f32(x), _f32(bias)
    if x.ndim < 2 or bias.ndim != 1 or x.shape[-1] != bias.shape[0]:
        raise InvalidArgument("addBias: expected [..., features] and [features]")
    return x + bias


def silu(x):
    x = _f32(x)
    return x / (F32(1.0) + np.exp(-x, dtype=F32))


def relu(x):
    x = _f32(x)
    return np.where(x > 0, x, F32(0.0)).astype(F32)


def gelu(x):
    x = _f32(x)
    inner = SQRT_2_OVER_PI * (x + GELU_COEFF * x * x * x)
    return F32(0.5) * x * (F32(1.0) + np.tanh(inner, dtype=F32))


# ---- matmul (src/backend/cpu/ops.cpp:161-181, 183-209) -------------------------------------------

def matmul(a, b, exact_order: bool = True):
    """[m,k] x [k,n]. exact_order=True reproduces the reference's i-p-j loop: every output element
    is a float32 running sum over p. exact_order=False uses a float64 dot (for larger cases where
    only a tolerance comparison is made)."""
    a, b = _f32(a), _f32(b)
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
        raise InvalidArgument("matmul: incompatible shapes")
    if not exact_order:
        return (a.astype(np.float64) @ b.astype(np.float64)).astype(F32)
    out = np.zeros((a.shape[0], b.shape[1]), dtype=F32)
    for p in range(a.shape[1]):
        out += a[:, p:p + 1] * b[p:p + 1, :]
    return out


def matmul_transpose_b(a, b, exact_order: bool = True):
    """[m,k] x [n,k]^T (src/backend/cpu/ops.cpp:183-209): float32 running sum over k."""
    a, b = _f32(a), _f32(b)
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[1]:
        raise InvalidArgument("matmulTransposeB: incompatible shapes")
    if not exact_order:
        return (a.astype(np.float64) @ b.astype(np.float64).T).astype(F32)
    out = np.zeros((a.shape[0], b.shape[0]), dtype=F32)
    for p in range(a.shape[1]):
        out += a[:, p:p + 1] * b[:, p][None, :]
    return out


def linear(x, w, bias, exact_order: bool = True):
    """src/backend/cpu/ops.cpp:226-248: flatten to [rows, in], matmul, addBias, restore shape."""
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    if x.ndim < 2:
        raise InvalidArgument("linear: rank >= 2 required")
    flat = x.reshape(-1, x.shape[-1])
    out = add_bias(matmul(flat, w, exact_order), bias)
    return out.reshape(x.shape[:-1] + (w.shape[1],))


# ---- rmsnorm / softmax (src/backend/cpu/ops.cpp:250-322) -----------------------------------------

def rmsnorm(x):
    """No gamma, eps 1e-6 added to the float64 mean square; rms cast to float32 before dividing."""
    x = _f32(x)
    if x.ndim < 2:
        raise InvalidArgument("rmsnorm: rank >= 2 required")
    rows = x.reshape(-1, x.shape[-1])
    acc = np.zeros(rows.shape[0], dtype=np.float64)
    for c in range(rows.shape[1]):
        v = rows[:, c].astype(np.float64)
        acc += v * v
    mean_sq = acc / np.float64(rows.shape[1])
    rms = np.sqrt(mean_sq + np.float64(RMS_EPS)).astype(F32)
    return (rows / rms[:, None]).astype(F32).reshape(x.shape)


def softmax(x):
    x = _f32(x)
    if x.ndim < 2:
        raise InvalidArgument("softmax: rank >= 2 required")
    rows = x.reshape(-1, x.shape[-1])
    mx = rows.max(axis=1, keepdims=True)
    e64 = np.exp((rows - mx).astype(np.float64))   # float32 subtraction, then double exp
    e32 = e64.astype(F32)
    total = np.zeros(rows.shape[0], dtype=np.float64)
    for c in range(rows.shape[1]):
        total += e64[:, c]
    out = (e32.astype(np.float64) / total[:, None]).astype(F32)
    return out.reshape(x.shape)


# ---- embedding / positions (src/backend/cpu/ops.cpp:324-425) -------------------------------------

def embedding_lookup(token_ids, table):
    """ids are float32 holding integers; lround (half away from zero); out-of-vocabulary throws."""
    ids, table = _f32(token_ids), _f32(table)
    if ids.ndim != 2 or table.ndim != 2:
        raise InvalidArgument("embeddingLookup: ids [batch, seq] and table [vocab, dim] required")
    idx = (np.sign(ids) * np.floor(np.abs(ids.astype(np.float64)) + 0.5)).astype(np.int64)
    if idx.size and (idx.min() < 0 or idx.max() >= table.shape[0]):
        raise InvalidArgument("embeddingLookup: token id outside the vocabulary")
    return table[idx]


def add_positional_embedding(x, table, offset: int = 0):
    x, table = _f32(x), _f32(table)
    if x.ndim != 3 or table.ndim != 2 or table.shape[1] != x.shape[2]:
        raise InvalidArgument("addPositionalEmbedding: input [batch, seq, dim], table [maxSeq, dim]")
    seq = x.shape[1]
    if offset + seq > table.shape[0]:
        raise InvalidArgument("addPositionalEmbedding: sequence exceeds maxSeqLen")
    return x + table[None, offset:offset + seq, :]


# ---- transformer blocks (src/backend/cpu/ops.cpp:427-495) ----------------------------------------

def feed_forward(x, w1, b1, w2, b2, gemm=None):
    gemm_linear = (lambda a, w, b: linear(a, w, b)) if gemm is None else gemm
    normed = rmsnorm(x)
    hidden = silu(gemm_linear(normed, w1, b1))
    return add(x, gemm_linear(hidden, w2, b2))


def attention_core(q, k, v, num_heads: int, causal: bool = True, old_len: int = 0, exact_order: bool = True):
    """softmax(scale * q k^T + mask) v per (batch, head); q [B,newLen,dim], k,v [B,totalLen,dim] with
    heads contiguous inside dim. Restates the per-head loop of src/backend/cpu/ops.cpp:476-488 and
    the incremental mask j <= oldLen + i of :98-109."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, new_len, dim = q.shape
    total_len = k.shape[1]
    hd = dim // num_heads
    factor = F32(1.0) / np.sqrt(F32(hd), dtype=F32)
    out = np.empty_like(q)
    for b in range(B):
        for h in range(num_heads):
            sl = slice(h * hd, (h + 1) * hd)
            scores = scale(matmul_transpose_b(q[b, :, sl], k[b, :, sl], exact_order), factor)
            if causal:
                i = np.arange(new_len)[:, None]
                j = np.arange(total_len)[None, :]
                scores = np.where(j > old_len + i, F32(-np.inf), scores).astype(F32)
            out[b, :, sl] = matmul(softmax(scores), v[b, :, sl], exact_order)
    return out


def attention_forward_stats(q, k, v, num_heads: int, scale_factor: float, old_len: int = 0):
    """(output, m, l) of the fused forward: m the row maximum of the scaled, masked scores and l the sum of
    exp(score - m), per (batch, head, query row) — the statistics the backward needs
    (src/backend/cuda/fused_attention.cu:56-156; the mask j <= oldLen + i of :96-99)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, new_len, dim = q.shape
    total_len = k.shape[1]
    hd = dim // num_heads
    out = np.zeros_like(q)
    m = np.zeros((B, num_heads, new_len), F32)
    l = np.zeros((B, num_heads, new_len), F32)
    i = np.arange(new_len)[:, None]
    j = np.arange(total_len)[None, :]
    for b in range(B):
        for h in range(num_heads):
            sl = slice(h * hd, (h + 1) * hd)
            s = (q[b, :, sl].astype(np.float64) @ k[b, :, sl].astype(np.float64).T) * float(scale_factor)
            s = np.where(j > old_len + i, -np.inf, s)
            mx = s.max(axis=1)
            e = np.exp(s - mx[:, None])
            lsum = e.sum(axis=1)
            out[b, :, sl] = ((e / lsum[:, None]) @ v[b, :, sl].astype(np.float64)).astype(F32)
            m[b, h], l[b, h] = mx.astype(F32), lsum.astype(F32)
    return out, m, l


def attention_backward(d_out, q, k, v, out, m, l, num_heads: int, scale_factor: float, old_len: int = 0):
    """(dQ, dK, dV) of the fused attention core, the arithmetic of fusedAttentionBackward
    (src/backend/cuda/fused_attention.cu:158-303): D_i = dot(out_i, dOut_i) (:166-190); per visible key j
    p = exp(score - m_i) / l_i, dP = dot(dOut_i, v_j), dScore = p (dP - D_i), dQ_i += dScore scale k_j,
    dK_j += dScore scale q_i, dV_j += p dOut_i (:255-296); keys no query row sees keep zero (:366-367).
    Accumulated in float64, so that it is the exact value both the reference's fp32 atomics and a tensor-core
    kernel approximate."""
    g, q, k, v, out = (np.asarray(t, dtype=np.float64) for t in (d_out, q, k, v, out))
    m, l = np.asarray(m, dtype=np.float64), np.asarray(l, dtype=np.float64)
    B, new_len, dim = q.shape
    total_len = k.shape[1]
    hd = dim // num_heads
    dq = np.zeros((B, new_len, dim), np.float64)
    dk = np.zeros((B, total_len, dim), np.float64)
    dv = np.zeros((B, total_len, dim), np.float64)
    i = np.arange(new_len)[:, None]
    j = np.arange(total_len)[None, :]
    visible = j <= old_len + i
    for b in range(B):
        for h in range(num_heads):
            sl = slice(h * hd, (h + 1) * hd)
            d_term = (out[b, :, sl] * g[b, :, sl]).sum(axis=1)
            s = (q[b, :, sl] @ k[b, :, sl].T) * float(scale_factor)
            with np.errstate(over="ignore"):
                p = np.where(visible, np.exp(np.where(visible, s, 0.0) - m[b, h][:, None]) / l[b, h][:, None], 0.0)
            dp = g[b, :, sl] @ v[b, :, sl].T
            ds = p * (dp - d_term[:, None]) * float(scale_factor)
            dq[b, :, sl] = ds @ k[b, :, sl]
            dk[b, :, sl] = ds.T @ q[b, :, sl]
            dv[b, :, sl] = p.T @ g[b, :, sl]
    return dq.astype(F32), dk.astype(F32), dv.astype(F32)


def self_attention(x, wq, wk, wv, wout, num_heads: int, causal: bool = True, gemm=None, exact_order: bool = True):
    x = _f32(x)
    if x.ndim != 3:
        raise InvalidArgument("selfAttention: input [batch, seq, dim] required")
    B, S, dim = x.shape
    if num_heads == 0 or dim % num_heads != 0:
        raise InvalidArgument("selfAttention: numHeads must divide dim")
    mm = (lambda a, w: matmul(a, w, exact_order)) if gemm is None else gemm
    normed = rmsnorm(x).reshape(B * S, dim)
    q = mm(normed, wq).reshape(B, S, dim)
    k = mm(normed, wk).reshape(B, S, dim)
    v = mm(normed, wv).reshape(B, S, dim)
    ctx = attention_core(q, k, v, num_heads, causal, 0, exact_order)
    proj = mm(ctx.reshape(B * S, dim), wout).reshape(B, S, dim)
    return add(x, proj)


# ---- simulated precision (src/backend/cpu/quantize.cpp:18-93) ------------------------------------

def round_bf16(x):
    x = _f32(x)
    bits = x.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(F32).copy()
    bad = ~np.isfinite(x)
    out[bad] = x[bad]
    return out


def _round_mantissa(x, mantissa_bits: int, max_mag: float):
    x = _f32(x)
    out = x.copy()
    live = np.isfinite(x) & (x != 0)
    mag = np.abs(x[live])
    sign = np.where(x[live] < 0, F32(-1), F32(1))
    mant, exp = np.frexp(mag)                      # mag = mant * 2^exp, mant in [0.5, 1)
    norm = (mant * F32(2.0)).astype(F32)
    sc = F32(1 << mantissa_bits)
    t = (norm * sc).astype(F32)
    rounded = (np.sign(t) * np.floor(np.abs(t) + F32(0.5))).astype(F32) / sc    # std::round
    bump = rounded >= 2.0
    rounded = np.where(bump, rounded * F32(0.5), rounded).astype(F32)
    exp = exp + bump.astype(exp.dtype)
    res = (sign * np.ldexp((rounded * F32(0.5)).astype(F32), exp)).astype(F32)
    res = np.where(np.abs(res) > F32(max_mag), sign * F32(max_mag), res).astype(F32)
    res = np.where(mag > F32(max_mag), sign * F32(max_mag), res).astype(F32)
    out[live] = res
    return out


def quantize(x, dtype: str):
    if dtype == "fp32":
        return _f32(x)
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "tf32":
        return _round_mantissa(x, 10, 3.4e38)
    if dtype == "fp16":
        return _round_mantissa(x, 10, 65504.0)
    if dtype == "fp8.e4m3":
        return _round_mantissa(x, 3, 448.0)
    if dtype == "fp8.e5m2":
        return _round_mantissa(x, 2, 57344.0)
    raise InvalidArgument(f"unknown dtype {dtype}")


def e4m3_round_hw(x):
    """Round to the real e4m3 grid as the GPU conversion does (round-to-nearest-even, saturate to
    +-448, subnormals down to 2^-9). The reference's simulated rounding above has no subnormals and
    rounds half away from zero; the two agree on normal values except at exact ties."""
    x = _f32(x).astype(np.float64)
    sign = np.sign(x)
    mag = np.minimum(np.abs(x), 448.0)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(mag > 0, mag, 1.0)))
    e = np.maximum(e, -6.0)                        # below 2^-6 the grid spacing stays 2^-9
    step = np.exp2(e - 3.0)
    q = np.round(mag / step) * step                # np.round = ties-to-even
    return (sign * np.minimum(q, 448.0)).astype(F32)


def fp8_scaled_matmul(a, w, exact_order: bool = False):
    """This project's definition of the `compute fp8.e4m3` GEMM (no counterpart in the reference):
    per-tensor scales s = 448 / amax, operands rounded to e4m3 after scaling, fp32 accumulate,
    result multiplied by 1 / (s_a * s_w)."""
    a, w = _f32(a), _f32(w)
    amax_a = np.max(np.abs(a)) if a.size else 0.0
    amax_w = np.max(np.abs(w)) if w.size else 0.0
    sa = F32(448.0) / F32(amax_a) if amax_a > 0 else F32(1.0)
    sw = F32(448.0) / F32(amax_w) if amax_w > 0 else F32(1.0)
    qa = e4m3_round_hw(a * sa)
    qw = e4m3_round_hw(w * sw)
    return (matmul(qa, qw, exact_order) * (F32(1.0) / (sa * sw))).astype(F32)


# ---- BFCKPT1 (include/blackforge/backend/cpu/checkpoint.hpp:15-24, src/backend/cpu/checkpoint.cpp) --

CKPT_MAGIC = b"BFCKPT1\x00"


def save_checkpoint(path: str, params: Sequence):
    """params: sequence of (name, float32 array). Little-endian u32/u64/fp32 as the reference writes."""
    with open(path, "wb") as f:
        f.write(CKPT_MAGIC)
        f.write(struct.pack("<I", len(params)))
        for name, value in params:
            value = _f32(value)
            nb = name.encode()
            f.write(struct.pack("<I", len(nb)))
            f.write(nb)
            f.write(struct.pack("<I", value.ndim))
            for d in value.shape:
                f.write(struct.pack("<Q", d))
            f.write(value.tobytes())


def load_checkpoint(path: str) -> List:
    try:
        f = open(path, "rb")
    except OSError as e:
        raise RuntimeFailure(f"loadCheckpoint: cannot open {path}") from e
    with f:
        if f.read(8) != CKPT_MAGIC:
            raise RuntimeFailure("loadCheckpoint: not a BlackForge checkpoint")
        (count,) = struct.unpack("<I", f.read(4))
        out = []
        for _ in range(count):
            hdr = f.read(4)
            if len(hdr) < 4:
                raise RuntimeFailure("loadCheckpoint: truncated")
            (nlen,) = struct.unpack("<I", hdr)
            name = f.read(nlen).decode()
            (rank,) = struct.unpack("<I", f.read(4))
            shape = [struct.unpack("<Q", f.read(8))[0] for _ in range(rank)]
            n = int(np.prod(shape)) if shape else 1
            raw = f.read(4 * n)
            if len(raw) != 4 * n:
                raise RuntimeFailure("loadCheckpoint: truncated")
            out.append((name, np.frombuffer(raw, dtype="<f4").reshape(shape).copy()))
        return out


# ---- model (src/backend/cpu/model.cpp:68-239) ----------------------------------------------------

def param_layout(ops: Sequence[dict], input_last_dim: Optional[int] = None) -> List:
    """Names and shapes of every parameter in checkpoint order. `ops` is the pipeline as dicts with
    keys kind/output/linear_out/vocab/emb_dim/max_seq/heads/hidden (mirror of ir::Operation,
    include/blackforge/ir/operation.hpp:23-33); the integer in a name is the op's output value id
    (src/backend/cpu/model.cpp:86, :112, :121, :143, :163)."""
    out = []
    feat = input_last_dim
    for op in ops:
        kind, oid = op["kind"], op["output"]
        if kind == "linear":
            out += [(f"linear{oid}.weight", (feat, op["linear_out"])), (f"linear{oid}.bias", (op["linear_out"],))]
            feat = op["linear_out"]
        elif kind == "embedding":
            out.append((f"embedding{oid}.table", (op["vocab"], op["emb_dim"])))
            feat = op["emb_dim"]
        elif kind == "positional_embedding":
            out.append((f"positional_embedding{oid}.table", (op["max_seq"], feat)))
        elif kind in ("attention", "bidirectional_attention"):
            if op["heads"] == 0 or feat % op["heads"] != 0:
                raise InvalidArgument("Model: heads must divide dim")
            out += [(f"{kind}{oid}.{s}", (feat, feat)) for s in ("wq", "wk", "wv", "wout")]
        elif kind == "feedforward":
            h = op["hidden"]
            out += [(f"feedforward{oid}.w1", (feat, h)), (f"feedforward{oid}.b1", (h,)),
                    (f"feedforward{oid}.w2", (h, feat)), (f"feedforward{oid}.b2", (feat,))]
    return out


def model_forward(ops: Sequence[dict], params: Dict[str, np.ndarray], x, cpu_policy: Optional[dict] = None,
                  cuda_policy: Optional[dict] = None, exact_order: bool = True, taps: Optional[dict] = None):
    """Forward of the pipeline. With cpu_policy={'storage','compute'} it follows cpu::Model::forward's
    simulated precision; with cuda_policy={'compute': 'bf16'|'fp8.e4m3'} it follows the CUDA meaning
    (every GEMM at `compute`, rest fp32). `taps`, if given, receives every op output by value id."""
    cur = _f32(x)
    if cpu_policy:
        cur = quantize(cur, cpu_policy["storage"])

    gemm_mm = None
    gemm_lin = None
    if cuda_policy and cuda_policy.get("compute") == "bf16":
        def gemm_mm(a, w):
            return matmul(round_bf16(a), round_bf16(w), exact_order)
    elif cuda_policy and cuda_policy.get("compute") == "fp8.e4m3":
        def gemm_mm(a, w):
            return fp8_scaled_matmul(a, w, exact_order)
    if gemm_mm is not None:
        def gemm_lin(a, w, b):
            flat = _f32(a).reshape(-1, a.shape[-1])
            return add_bias(gemm_mm(flat, w), b).reshape(a.shape[:-1] + (w.shape[1],))

    for op in ops:
        kind, oid = op["kind"], op["output"]
        if kind == "linear":
            w, b = params[f"linear{oid}.weight"], params[f"linear{oid}.bias"]
            if cpu_policy:
                cur = linear(quantize(cur, cpu_policy["compute"]), quantize(w, cpu_policy["compute"]), b, exact_order)
            elif gemm_lin is not None:
                cur = gemm_lin(cur, w, b)
            else:
                cur = linear(cur, w, b, exact_order)
        elif kind == "silu":
            cur = silu(cur)
        elif kind == "relu":
            cur = relu(cur)
        elif kind == "gelu":
            cur = gelu(cur)
        elif kind == "rmsnorm":
            cur = rmsnorm(cur)
        elif kind == "softmax":
            cur = softmax(cur)
        elif kind == "embedding":
            cur = embedding_lookup(cur, params[f"embedding{oid}.table"])
        elif kind == "positional_embedding":
            cur = add_positional_embedding(cur, params[f"positional_embedding{oid}.table"])
        elif kind in ("attention", "bidirectional_attention"):
            p = [params[f"{kind}{oid}.{s}"] for s in ("wq", "wk", "wv", "wout")]
            cur = self_attention(cur, *p, op["heads"], causal=(kind == "attention"), gemm=gemm_mm,
                                 exact_order=exact_order)
        elif kind == "feedforward":
            p = [params[f"feedforward{oid}.{s}"] for s in ("w1", "b1", "w2", "b2")]
            cur = feed_forward(cur, *p, gemm=gemm_lin if gemm_lin is not None else
                               (lambda a, w, b: linear(a, w, b, exact_order)))
        else:
            raise InvalidArgument(f"unknown op {kind}")
        if cpu_policy:
            cur = quantize(cur, cpu_policy["storage"])
        if taps is not None:
            taps[oid] = cur
    return cur


# ---- seeded synthetic inputs (this project's generators, not the reference's) --------------------

def synth_params(ops: Sequence[dict], input_last_dim: Optional[int], seed: int, sigma: float,
                 bias_sigma: Optional[float] = None) -> Dict[str, np.ndarray]:
    """N(0, sigma) weights and biases from numpy's PCG64, one independent stream per parameter
    (seed, index). Stands in for a trained checkpoint; written to BFCKPT1 for both sides."""
    out = {}
    for i, (name, shape) in enumerate(param_layout(ops, input_last_dim)):
        rng = np.random.Generator(np.random.PCG64([seed, i]))
        s = sigma if len(shape) > 1 or bias_sigma is None else bias_sigma
        out[name] = (rng.standard_normal(shape, dtype=F32) * F32(s)).astype(F32)
    return out


def synth_token_ids(batch: int, seq: int, vocab: int, seed: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64([seed, 0xB0B]))
    return rng.integers(0, vocab, size=(batch, seq)).astype(F32)


def lm_ops(vocab: int, dim: int, layers: int, heads: int, hidden: int, max_seq: int) -> List[dict]:
    """The decoder-only pipeline `embedding |> positional_embedding |> (attention |> feedforward)*L |>
    linear(vocab)` with value ids numbered from 1 as the reference's IR builder does."""
    ops, vid = [], 0

    def push(kind, **kw):
        nonlocal vid
        base = {"kind": kind, "input": vid, "output": vid + 1, "linear_out": 0, "vocab": 0, "emb_dim": 0,
                "max_seq": 0, "heads": 0, "hidden": 0}
        base.update(kw)
        ops.append(base)
        vid += 1

    push("embedding", vocab=vocab, emb_dim=dim)
    push("positional_embedding", max_seq=max_seq)
    for _ in range(layers):
        push("attention", heads=heads)
        push("feedforward", hidden=hidden)
    push("linear", linear_out=vocab)
    return ops


def lm_source(vocab: int, dim: int, layers: int, heads: int, hidden: int, max_seq: int, seq: int,
              precision: Optional[dict] = None, name: str = "LM") -> str:
    """The same pipeline as BlackForge source text (grammar: docs/language.md:84-129)."""
    stages = [f"embedding({vocab}, {dim})", f"positional_embedding({max_seq})"]
    for _ in range(layers):
        stages += [f"attention({heads})", f"feedforward({hidden})"]
    stages.append(f"linear({vocab})")
    head = ""
    if precision:
        head = "precision {\n" + "".join(f"    {k} {v}\n" for k, v in precision.items()) + "}\n"
    return f"{head}model {name} {{\n    input fp32[batch, {seq}]\n    input |> " + " |> ".join(stages) + "\n}\n"
