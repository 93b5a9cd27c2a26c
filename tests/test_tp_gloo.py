"""The tensor-parallel plan on CPU ranks (gloo, world size 2): the slices that
vx_b200.llama.tp_slices hands each rank, combined the way the decoder combines
them (partial output/down projections summed across ranks, vocabulary-split
logits reduced to a best (value, index)), must give what the unsharded oracle
gives."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(dim=128, hidden=352, q_heads=4, kv_heads=2, head_dim=32, vocab=512)
POS = 5


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def model(oracle):
    c = CFG
    qkv_rows = (c["q_heads"] + 2 * c["kv_heads"]) * c["head_dim"]

    def w(n, seed):
        return oracle.f32_to_bf16(oracle.random_f32(n, seed, 0.1))

    return dict(wqkv=w(qkv_rows * c["dim"], 1).reshape(qkv_rows, c["dim"]),
                wo=w(c["dim"] * c["q_heads"] * c["head_dim"], 2).reshape(c["dim"], -1),
                wgu=w(2 * c["hidden"] * c["dim"], 3).reshape(2 * c["hidden"], c["dim"]),
                wd=w(c["dim"] * c["hidden"], 4).reshape(c["dim"], c["hidden"]),
                head=w(c["vocab"] * c["dim"], 5).reshape(c["vocab"], c["dim"]),
                norm=oracle.f32_to_bf16(np.ones(c["dim"], np.float32)),
                x=oracle.random_f32(c["dim"], 6, 1.0),
                kc=oracle.random_f32(8 * c["kv_heads"] * c["head_dim"], 7, 1.0)
                .reshape(8, c["kv_heads"], c["head_dim"]),
                vc=oracle.random_f32(8 * c["kv_heads"] * c["head_dim"], 8, 1.0)
                .reshape(8, c["kv_heads"], c["head_dim"]))


def layer(oracle, m, rank, ranks, reduce_sum, best_of):
    """One decoder layer + classifier on rank's slices. reduce_sum adds a
    [dim] vector across ranks; best_of picks the best (value, index)."""
    from vx_b200.llama import tp_slices
    c = CFG
    hd = c["head_dim"]
    sl = tp_slices(c["q_heads"], c["kv_heads"], hd, c["hidden"], c["vocab"],
                   rank, ranks)
    ql, kvl, hl = sl["q_local"], sl["kv_local"], sl["hidden_local"]
    cos, sin = oracle.rope_tables(8, hd, 10000.0)
    x = m["x"].copy()
    xb = oracle.nn_rms_norm(x, m["norm"], c["dim"], 1e-5)
    w_local = np.ascontiguousarray(np.concatenate(
        [m["wqkv"][slice(*sl[k])] for k in ("q_rows", "k_rows", "v_rows")]))
    bias = np.zeros(w_local.shape[0], np.uint16)
    q, k, v = oracle.nn_qkv(w_local, bias, xb, ql, kvl, hd, c["dim"])
    g0 = rank * kvl
    kc = np.ascontiguousarray(m["kc"][:, g0:g0 + kvl])
    vc = np.ascontiguousarray(m["vc"][:, g0:g0 + kvl])
    qr = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, POS)
    att = oracle.nn_attention(qr, kc, vc, POS)
    wo = np.ascontiguousarray(m["wo"][:, slice(*sl["wo_cols"])])
    part = oracle.nn_matvec(wo, att.reshape(-1), c["dim"], ql * hd)
    x = x + reduce_sum(part)
    xb = oracle.nn_rms_norm(x, m["norm"], c["dim"], 1e-5)
    wgu = np.ascontiguousarray(np.concatenate(
        [m["wgu"][slice(*sl["gate_rows"])], m["wgu"][slice(*sl["up_rows"])]]))
    h = oracle.nn_swiglu(wgu, xb, hl, c["dim"])
    wd = np.ascontiguousarray(m["wd"][:, slice(*sl["down_cols"])])
    x = x + reduce_sum(oracle.nn_matvec(wd, h, c["dim"], hl))
    xb = oracle.nn_rms_norm(x, m["norm"], c["dim"], 1e-5)
    head = np.ascontiguousarray(m["head"][slice(*sl["vocab_rows"])])
    logits = oracle.nn_matvec(head, xb, sl["vocab_local"], c["dim"])
    i = oracle.nn_argmax(logits)
    return x, best_of(float(logits[i]), i + sl["vocab_rows"][0])


def worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import vx_oracle as oracle
    oracle.set_threads(1)

    def reduce_sum(v):
        t = torch.from_numpy(v.astype(np.float32))
        dist.all_reduce(t)
        return t.numpy()

    def best_of(value, index):
        mine = torch.tensor([value, float(index)], dtype=torch.float64)
        every = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(every, mine)
        best = every[0]
        for p in every[1:]:                 # rank order is index order
            if p[0] > best[0]:
                best = p
        return int(best[1])

    x, token = layer(oracle, model(oracle), rank, world, reduce_sum, best_of)
    if rank == 0:
        np.save(out, np.concatenate([x, [token]]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_give_the_unsharded_result(oracle, tmp_path):
    out = str(tmp_path / "tp.npy")
    mp.spawn(worker, args=(2, free_port(), out), nprocs=2, join=True)
    got = np.load(out)
    want_x, want_token = layer(oracle, model(oracle), 0, 1, lambda v: v,
                               lambda value, index: index)
    # partial sums are added in a different order: rounding-level difference
    assert np.abs(got[:-1] - want_x).max() <= 1e-5 * np.abs(want_x).max()
    assert int(got[-1]) == want_token


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
def test_slices_tile_every_matrix_exactly(ranks):
    from vx_b200.llama import LLAMA2_7B, tp_slices
    s = LLAMA2_7B
    args = (s["q_heads"], s["kv_heads"], s["head_dim"], s["hidden"], s["vocab"])
    for key, total, first in [("q_rows", s["q_heads"] * 128, 0),
                              ("k_rows", s["kv_heads"] * 128, s["q_heads"] * 128),
                              ("gate_rows", s["hidden"], 0),
                              ("up_rows", s["hidden"], s["hidden"]),
                              ("wo_cols", s["q_heads"] * 128, 0),
                              ("down_cols", s["hidden"], 0),
                              ("vocab_rows", s["vocab"], 0)]:
        at = first
        for r in range(ranks):
            lo, hi = tp_slices(*args, r, ranks)[key]
            assert lo == at and hi > lo
            at = hi
        assert at == first + total
