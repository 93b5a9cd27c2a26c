"""Run under torchrun by tests/test_gpu_tp.py: the column-split product
(local GEMM, all-gather over the job, interleave) against the whole product
computed by rank 0 alone."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from vx_b200 import abi, collective, ops  # noqa: E402
from vx_b200.lib import check, lib  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    here = abi.gpu(local)  # this rank's tensors live on its own GPU
    collective.join_job(rank, world)
    m, n, k = 384, 512 * world, 640
    nl = n // world
    rng = np.random.default_rng(3)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-2, 3, (k, n)).astype(np.float32)
    bf = lambda x: (x.view(np.uint32) >> 16).astype(np.uint16)  # exact: small integers
    ta = abi.DeviceTensor.from_host(bf(a), topo=here, bf16=True)
    tb = abi.DeviceTensor.from_host(bf(np.ascontiguousarray(b[:, rank * nl:(rank + 1) * nl])), topo=here, bf16=True)
    tcl = abi.DeviceTensor.empty((m, nl), abi.BF16, here)
    tg = abi.DeviceTensor.empty((world, m, nl), abi.BF16, here)
    tc = abi.DeviceTensor.empty((m, n), abi.BF16, here)
    check(lib().vx_b200_gemm_column_split(abi.BF16, m, nl, k, ta.ptr, tb.ptr,
                                          tcl.ptr, tg.ptr, tc.ptr))
    got = tc.to_host()
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    want = ((exact.view(np.uint32) + 0x7FFF + ((exact.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    status = ops.kernel_status()
    assert status == 0, "rank %d: kernel status 0x%x" % (rank, status)
    assert np.array_equal(got, want), "rank %d: column-split product differs" % rank
    collective.leave_job()


if __name__ == "__main__":
    main()
