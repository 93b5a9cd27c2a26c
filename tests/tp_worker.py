"""Run under torchrun by tests/test_gpu_tp.py: every rank builds its slice of a
small std::nn model, decodes a prompt and greedy steps with the tensor-parallel
decoder, and rank 0 writes the tokens; with one rank it is the unsharded run."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from vx_b200 import collective, llama  # noqa: E402

SHAPE = dict(dim=512, hidden=1408, n_layers=4, q_heads=8, kv_heads=4,
             head_dim=64, vocab=4096)
BATCH = 2
if os.environ.get("VX_TEST_TP_SHAPE") == "one_launch":
    # one sequence and heads of 128 values: the step is one cooperative launch
    SHAPE = dict(SHAPE, head_dim=128)
    BATCH = 1


def main():
    out = sys.argv[1]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        collective.join_job(rank, world)
    dec, _ = llama.nn_bf16_model(max_seq=96, batch=BATCH, tp_rank=rank,
                                 tp_ranks=world,
                                 tp_reduce=int(os.environ.get("VX_TEST_TP_REDUCE", "1")),
                                 **SHAPE)
    prompts = np.random.default_rng(8).integers(0, SHAPE["vocab"], (BATCH, 24))
    tokens = []
    for p in range(prompts.shape[1]):
        toks = dec.step(list(prompts[:, p]))
    for _ in range(24):
        tokens.append(list(toks))
        toks = dec.step(None)
    per_step = dec.kernels_per_step
    dec.close()
    if BATCH == 1:
        assert per_step <= 6, "the step did not run as one launch"
    from vx_b200 import ops
    assert ops.kernel_status() == 0, "a bounded wait gave up"
    if world > 1:
        collective.leave_job()
    if rank == 0:
        with open(out, "w") as f:
            json.dump(tokens, f)


if __name__ == "__main__":
    main()
