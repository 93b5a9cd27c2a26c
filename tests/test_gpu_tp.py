"""Tensor-parallel decoding on two GPUs must give the tokens of one GPU: one
process per GPU, joined by vx_collective_init through VX_NCCL_ID_FILE, partial
projections summed by the NCCL all-reduce inside the token graph."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "tp_worker.py")


def gpu_count():
    import torch
    return torch.cuda.device_count()


def run(world, out, tmp_path, reduce=1, shape=""):
    env = dict(os.environ)
    env["VX_TEST_TP_REDUCE"] = str(reduce)
    env["VX_TEST_TP_SHAPE"] = shape
    if shape == "one_launch":
        env["VXB_STEP_KERNEL"] = "1"
    if world == 1:
        cmd = [sys.executable, WORKER, out]
    else:
        id_file = str(tmp_path / ("nccl_id_%d" % reduce))
        env["VX_NCCL_ID_FILE"] = id_file
        env["NCCL_NVLS_ENABLE"] = "0"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
               "--master-port", "29611", WORKER, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    with open(out) as f:
        return json.load(f)


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_decode_the_tokens_of_one(tmp_path):
    one = run(1, str(tmp_path / "one.json"), tmp_path)
    pushed = run(2, str(tmp_path / "two.json"), tmp_path, reduce=1)
    nccl = run(2, str(tmp_path / "two_nccl.json"), tmp_path, reduce=0)
    assert one == pushed, "partials pushed through peer memory"
    assert one == nccl, "partials summed by NCCL"


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_with_the_step_as_one_launch(tmp_path):
    """One sequence: every rank runs its slice of the step as one cooperative
    launch, and the partial sums cross inside it."""
    one = run(1, str(tmp_path / "one.json"), tmp_path, shape="one_launch")
    two = run(2, str(tmp_path / "two.json"), tmp_path, shape="one_launch")
    assert one == two


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_column_split_gemm_with_all_gather(tmp_path):
    env = dict(os.environ)
    env["VX_NCCL_ID_FILE"] = str(tmp_path / "nccl_id_gemm")
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29612",
           os.path.join(ROOT, "tests", "gemm_tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_one_process_uses_two_gpus_in_turn():
    """`spawn on(Topology::GPU[i])` switches GPUs inside one process: kernels
    that opt in to more than 48 KiB of shared memory (the projections' weight
    ring, the tensor-core GEMMs) must get that opt-in on every GPU they run
    on, not only on the first."""
    code = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, %r)
from oracle import vx_oracle as oracle
from vx_b200 import abi, ops
rng = np.random.default_rng(0)
a16 = oracle.f32_to_bf16(rng.uniform(-1, 1, (512, 256)).astype(np.float32))
b16 = oracle.f32_to_bf16(rng.uniform(-1, 1, (256, 512)).astype(np.float32))
w = oracle.f32_to_bf16(oracle.random_f32(2 * 200 * 896, 41, 0.1))
x = oracle.random_f32(896, 42, 1.0)
want_c = oracle.bf16_to_f32(oracle.gemm_bf16_rows(a16, b16, np.arange(512)))
want_s = oracle.nn_swiglu(w, x, 200, 896)
for g in (0, 1, 0):
    torch.cuda.set_device(g)
    abi.set_home_gpu(g)
    ta = abi.DeviceTensor.from_host(a16, bf16=True)
    tb = abi.DeviceTensor.from_host(b16, bf16=True)
    got = oracle.bf16_to_f32(ops.matmul(ta, tb).to_host())
    assert np.linalg.norm(got - want_c) <= 4e-3 * np.linalg.norm(want_c), g
    out = abi.DeviceTensor.empty((200,), abi.F32)
    ops.nn_swiglu(out, abi.DeviceTensor.from_host(w, bf16=True),
                  abi.DeviceTensor.from_host(x), 200, 896)
    assert np.abs(out.to_host() - want_s).max() <= 2e-5 * np.abs(want_s).max(), g
    assert ops.kernel_status() == 0
print("both GPUs ok")
""" % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "both GPUs ok" in r.stdout, r.stderr[-3000:]


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_kv_cache_handed_from_gpu_0_to_gpu_1():
    """Prefill on GPU 0, decode on GPU 1 (handoff_kv, tests/backend/pass/
    llama2.vx:431-458): the caches cross with vx_plugin_transfer_peer, and the
    decoder on GPU 1 continues with the tokens of a single decoder."""
    code = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, %r)
from vx_b200 import abi, llama, ops
from vx_b200.lib import lib
shape = dict(dim=512, hidden=1408, n_layers=4, q_heads=8, kv_heads=4, head_dim=64, vocab=4096)
prompt = [int(t) for t in np.random.default_rng(12).integers(0, 4096, 30)]
def tokens_after(dec, first, n=20):
    out, tok = [], first
    for _ in range(n):
        out.append(tok)
        tok = dec.step([tok])[0]
    return out
torch.cuda.set_device(0); abi.set_home_gpu(0)
pre, _ = llama.nn_bf16_model(max_seq=96, batch=1, **shape)
for t in prompt[:-1]:
    pre.step([t], fetch=False)
first = pre.step([prompt[-1]])[0]
nbytes = pre.kv_cache_bytes
k = lib().vx_plugin_transfer_peer(pre.kv_cache(0), abi.gpu(0), abi.gpu(1), nbytes)
v = lib().vx_plugin_transfer_peer(pre.kv_cache(1), abi.gpu(0), abi.gpu(1), nbytes)
want = tokens_after(pre, first)
pre.close()
torch.cuda.set_device(1); abi.set_home_gpu(1)
dec, _ = llama.nn_bf16_model(max_seq=96, batch=1, **shape)
dec.adopt_kv(k, v, len(prompt))
got = tokens_after(dec, first)
lib().vx_plugin_free(k, abi.gpu(1)); lib().vx_plugin_free(v, abi.gpu(1))
dec.close()
assert ops.kernel_status() == 0
assert got == want, (got, want)
print("handed over")
""" % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "handed over" in r.stdout, r.stderr[-3000:]
