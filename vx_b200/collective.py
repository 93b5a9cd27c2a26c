"""stdlib/std/collective.vx:35-79 over the eight vx_collective_* calls."""
import os

from . import abi
from .lib import lib


def join_job(rank, ranks):
    """Join the job (one process per GPU). Under a launcher that sets
    LOCAL_RANK, tensors made without an explicit topology go to that GPU from
    here on."""
    if "LOCAL_RANK" in os.environ:
        abi.set_home_gpu(int(os.environ["LOCAL_RANK"]))
    lib().vx_collective_init(rank, ranks)


def leave_job():
    lib().vx_collective_finish()


def job_rank():
    return lib().vx_collective_rank()


def job_ranks():
    return lib().vx_collective_ranks()


def all_reduce_sum(t):
    """In place, f32 or bf16."""
    fn = (lib().vx_collective_all_reduce_sum_bf16 if t.elem == abi.BF16
          else lib().vx_collective_all_reduce_sum_f32)
    fn(t.ptr, t.ptr, t.count)


def all_gather(t, out):
    assert out.count == t.count * max(job_ranks(), 1), \
        "all_gather: out.len must be in.len * ranks"
    fn = (lib().vx_collective_all_gather_bf16 if t.elem == abi.BF16
          else lib().vx_collective_all_gather_f32)
    fn(t.ptr, out.ptr, t.count)
