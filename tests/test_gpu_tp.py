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


def run(world, out, tmp_path, reduce=1):
    env = dict(os.environ)
    env["VX_TEST_TP_REDUCE"] = str(reduce)
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
