"""Tensor parallelism over two GPUs (heads, feed-forward columns and logits columns sharded, NCCL all-reduce
after the out-projection and the feed-forward down-projection) against the one-GPU result. Runs as two child
processes, one per GPU; skipped on a one-GPU box."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import bf_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(vocab=512, dim=512, layers=2, heads=4, hidden=1024, max_seq=160)

WORKER = r"""
import os, sys, time
import numpy as np
sys.path.insert(0, os.environ["BFB_ROOT"])
import blackforge_b200 as bfb
from oracle import bf_oracle as O
rank, world, work = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
cfg = eval(sys.argv[4])
bfb.check(bfb.lib().bfb_set_device(rank))
id_path = os.path.join(work, "nccl_id")
if rank == 0:
    ident = bfb.tp_unique_id()
    with open(id_path + ".tmp", "wb") as f:
        f.write(ident)
    os.replace(id_path + ".tmp", id_path)
else:
    deadline = time.time() + 120
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise SystemExit("no communicator id from rank 0")
        time.sleep(0.05)
    ident = open(id_path, "rb").read()
bfb.tp_init(ident, rank, world)
ops = O.lm_ops(**cfg)
params = O.synth_params(ops, None, seed=21, sigma=0.05, bias_sigma=0.05)
ids = O.synth_token_ids(2, 160, cfg["vocab"], seed=22)
m = bfb.Model(ops, precision={"storage": "fp32", "compute": "bf16"}, random_init=False)
m.set_tensor_parallel(rank, world)
m.set_params(params)
out = m.forward_host(ids)
np.save(os.path.join(work, f"logits_{rank}.npy"), out)
# the same pass with the all-reduces on the caller's stream (no sequence groups), and with other settings: the
# groups are independent sequences and a two-rank sum has one order, so every value is the same
for groups, reserved in ((1, 0), (2, 0), (2, 32)):
    m.set_tensor_parallel_overlap(groups, reserved)
    again = m.forward_host(ids)
    assert np.array_equal(again, out), (groups, reserved, float(np.max(np.abs(again - out))))
# the same weights from a checkpoint file: each rank streams its own slices (row ranges read directly, column
# slices cut out of full rows by the upload)
ckpt = os.path.join(work, f"weights_{rank}.bfckpt")
O.save_checkpoint(ckpt, [(n, params[n]) for n, _ in O.param_layout(ops)])
mc = bfb.Model(ops, precision={"storage": "fp32", "compute": "bf16"}, random_init=False)
mc.set_tensor_parallel(rank, world)
stats = mc.load_checkpoint_streaming(ckpt, 8192)
assert stats["read_bytes"] < stats["file_bytes"] and stats["uploaded_bytes"] < stats["read_bytes"], stats
assert np.array_equal(mc.forward_host(ids), out)
mc.close()
# bf16 residual stream (rmsnorm folded into the GEMMs, statistics per group)
m16 = bfb.Model(ops, precision={"storage": "bf16", "compute": "bf16"}, random_init=False)
m16.set_tensor_parallel(rank, world)
m16.set_params(params)
ids4 = O.synth_token_ids(4, 160, cfg["vocab"], seed=23)
m16.set_tensor_parallel_overlap(1, 0)
plain = m16.forward_host(ids4)
m16.set_tensor_parallel_overlap(2, 16)
grouped = m16.forward_host(ids4)
assert np.array_equal(plain, grouped), float(np.max(np.abs(plain - grouped)))
np.save(os.path.join(work, f"logits16_{rank}.npy"), grouped)
# e4m3 operands with four sequence groups: every group quantises its own GEMM inputs, so the pass needs a block of
# scales per group and layer (per-tensor scales follow the group, so the values differ a little from one group)
m8 = bfb.Model(ops, precision={"storage": "bf16", "compute": "fp8.e4m3"}, random_init=False)
m8.set_tensor_parallel(rank, world)
m8.set_params(params)
m8.set_tensor_parallel_overlap(4, 0)
np.save(os.path.join(work, f"logits8_{rank}.npy"), m8.forward_host(ids4))
bfb.tp_destroy()
print("rank", rank, "ok", out.shape)
"""


def test_two_gpu_tensor_parallel_matches_single_gpu(gpu, tmp_path):
    n = C.c_int32(0)
    gpu.check(gpu.lib().bfb_device_count(C.byref(n)))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, BFB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path), repr(CFG)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    parts = [np.load(tmp_path / f"logits_{r}.npy") for r in range(2)]
    assert parts[0].shape == (2, 160, CFG["vocab"] // 2)
    sharded = np.concatenate(parts, axis=-1)
    ops = O.lm_ops(**CFG)
    params = O.synth_params(ops, None, seed=21, sigma=0.05, bias_sigma=0.05)
    ids = O.synth_token_ids(2, 160, CFG["vocab"], seed=22)
    single = gpu.Model(ops, precision={"storage": "fp32", "compute": "bf16"}, random_init=False)
    single.set_params(params)
    want = single.forward_host(ids)
    # same arithmetic, different summation order across the two partial products
    assert np.max(np.abs(sharded - want)) / np.max(np.abs(want)) <= 5e-3
    # and against the oracle's statement of the reference's bf16 device path (bf16 GEMM operands, fp32 elsewhere)
    oracle = O.model_forward(ops, params, ids, cuda_policy={"compute": "bf16"}, exact_order=False)
    assert np.max(np.abs(sharded - oracle)) / np.max(np.abs(oracle)) <= 2e-2
    # bf16 residual stream, four sequences in two groups
    sharded16 = np.concatenate([np.load(tmp_path / f"logits16_{r}.npy") for r in range(2)], axis=-1)
    single16 = gpu.Model(ops, precision={"storage": "bf16", "compute": "bf16"}, random_init=False)
    single16.set_params(params)
    want16 = single16.forward_host(O.synth_token_ids(4, 160, CFG["vocab"], seed=23))
    assert np.sqrt(np.sum((sharded16 - want16) ** 2) / np.sum(want16 ** 2)) <= 2e-2
    # e4m3 operands, four groups: finite and within the e4m3 tolerance of the bf16 result
    sharded8 = np.concatenate([np.load(tmp_path / f"logits8_{r}.npy") for r in range(2)], axis=-1)
    assert np.isfinite(sharded8).all()
    assert np.sqrt(np.sum((sharded8 - want16) ** 2) / np.sum(want16 ** 2)) <= 0.15


GRAD_WORKER = r"""
import ctypes as C
import os, sys, time
import numpy as np
sys.path.insert(0, os.environ["BFB_ROOT"])
import blackforge_b200 as bfb
rank, world, work = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
bfb.check(bfb.lib().bfb_set_device(rank))
id_path = os.path.join(work, "nccl_id_grad")
if rank == 0:
    ident = bfb.tp_unique_id()
    with open(id_path + ".tmp", "wb") as f:
        f.write(ident)
    os.replace(id_path + ".tmp", id_path)
else:
    deadline = time.time() + 120
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise SystemExit("no communicator id from rank 0")
        time.sleep(0.05)
    ident = open(id_path, "rb").read()
bfb.tp_init(ident, rank, world)
# every replica's own gradients: a large matrix, ragged small tensors and an empty one, seeded by the rank
shapes = [(1024, 1536), (1536,), (7,), (0,), (3, 5)]
rng = np.random.default_rng(100 + rank)
grads = [rng.standard_normal(s).astype(np.float32) for s in shapes]
bufs = [bfb.upload(g, bfb.F32) for g in grads]
table = (C.c_void_p * len(bufs))(*[b.ptr or None for b in bufs])
counts = (C.c_int64 * len(bufs))(*[g.size for g in grads])
bfb.check(bfb.lib().bfb_gradients_average(table, counts, len(bufs), None))
bfb.sync()
for i, (b, s) in enumerate(zip(bufs, shapes)):
    np.save(os.path.join(work, f"avg_{rank}_{i}.npy"), bfb.download(b, bfb.F32, s))
bfb.tp_destroy()
print("rank", rank, "ok")
"""


def test_two_gpu_gradient_average_matches_the_host_staged_average(gpu, tmp_path):
    """The grouped NCCL average against the reference's rule (multi_gpu_train_runner.cu:275-297): the replicas'
    gradients added in replica order and scaled by 1 / replicas; with two replicas both give the same bits, and
    every replica ends with the same values."""
    n = C.c_int32(0)
    gpu.check(gpu.lib().bfb_device_count(C.byref(n)))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "grad_worker.py"
    script.write_text(GRAD_WORKER)
    env = dict(os.environ, BFB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    shapes = [(1024, 1536), (1536,), (7,), (0,), (3, 5)]
    rngs = [np.random.default_rng(100 + r) for r in range(2)]
    per_rank = [[rng.standard_normal(s).astype(np.float32) for s in shapes] for rng in rngs]
    for i, s in enumerate(shapes):
        want = O.scale(O.add(per_rank[0][i], per_rank[1][i]), np.float32(0.5)) if np.prod(s) else np.zeros(s, np.float32)
        got = [np.load(tmp_path / f"avg_{r}_{i}.npy") for r in range(2)]
        assert np.array_equal(got[0], got[1]) and np.array_equal(got[0], want), i


def test_gradient_average_without_a_communicator_is_refused(gpu):
    buf = gpu.DeviceBuffer.zeros(16)
    table = (C.c_void_p * 1)(buf.ptr)
    counts = (C.c_int64 * 1)(4)
    assert gpu.lib().bfb_gradients_average(table, counts, 1, None) == gpu.INVALID_ARGUMENT


ONE_RANK_WORKER = r"""
import ctypes as C
import os, sys
import numpy as np
sys.path.insert(0, os.environ["BFB_ROOT"])
import blackforge_b200 as bfb
bfb.check(bfb.lib().bfb_set_device(0))
bfb.tp_init(bfb.tp_unique_id(), 0, 1)
rng = np.random.default_rng(9)
grads = [rng.standard_normal(s).astype(np.float32) for s in ((257, 33), (5,), (0,))]
bufs = [bfb.upload(g, bfb.F32) for g in grads]
table = (C.c_void_p * len(bufs))(*[b.ptr or None for b in bufs])
counts = (C.c_int64 * len(bufs))(*[g.size for g in grads])
bfb.check(bfb.lib().bfb_gradients_average(table, counts, len(bufs), None))
bfb.sync()
for b, g in zip(bufs, grads):
    assert np.array_equal(bfb.download(b, bfb.F32, g.shape), g)
# a negative count is refused before anything is issued
bad = (C.c_int64 * 1)(-1)
assert bfb.lib().bfb_gradients_average(table, bad, 1, None) == bfb.INVALID_ARGUMENT
bfb.tp_destroy()
print("one rank ok")
"""


def test_gradient_average_over_one_replica_is_the_identity(gpu, tmp_path):
    """The grouped average on a one-rank communicator (what a single-GPU box can run): every gradient comes back
    unchanged, an empty tensor is skipped, a bad table is refused."""
    script = tmp_path / "one_rank_worker.py"
    script.write_text(ONE_RANK_WORKER)
    env = dict(os.environ, BFB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=300)
    assert proc.returncode == 0 and "one rank ok" in proc.stdout, proc.stdout
