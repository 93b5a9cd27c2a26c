"""Small, self-timing runs of one kernel each, for profiling a kernel on a case
that ends quickly (a few launches, at most a few GB on the device, inputs
larger than the 126 MB L2 where DRAM figures matter).

  python microbench.py rowdot  [--layers 4] [--iters 3]
  python microbench.py gemm    [--n 4096] [--iters 3] [--fmt bf16|f32|q4|fp8]
  python microbench.py flash   [--batch 1] [--heads 8] [--seq 4096]
  python microbench.py attn    [--pos 600]
  python microbench.py shard   [--ranks 8] [--pos 520]
  python microbench.py prefill [--layers 4] [--fmt bf16|q4|fp8]
  python microbench.py moe     [--n 512]
Each prints one JSON line with the CUDA-event time per launch.
"""
import argparse
import ctypes as C
import json

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from vx_b200 import abi, ops  # noqa: E402
from vx_b200.lib import lib  # noqa: E402


def _timed(torch, stream, fn, iters):
    lib().vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    try:
        fn()
        stream.synchronize()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            fn()
        b.record(stream)
        b.synchronize()
        return a.elapsed_time(b) / iters
    finally:
        lib().vx_cuda_set_stream(None)


def rowdot(torch, args):
    """The gate/up projection + SwiGLU at Llama-2-7B shapes over `layers`
    different matrices (180 MB each in bf16; --fmt fp8 or q4: the same matrix
    quantised, 90 or 51 MB)."""
    import torch as th
    dim, hid = 4096, 11008
    x = abi.DeviceTensor.empty((dim,), abi.F32)
    ops.fill_normal(x, 99, 1.0)
    out = abi.DeviceTensor.empty((hid,), abi.F32)
    if args.fmt == "bf16":
        ws = [abi.DeviceTensor.empty((2 * hid * dim,), abi.BF16)
              for _ in range(args.layers)]
        for i, w in enumerate(ws):
            ops.fill_normal(w, 100 + i, 0.02)
        run = lambda: [ops.nn_swiglu(out, w, x, hid, dim) for w in ws]
        nbytes = 2 * hid * dim * 2 + dim * 4 + hid * 4
    else:
        code = 2 if args.fmt == "fp8" else 3
        per = 2 * hid * dim
        quantised = []
        src = abi.DeviceTensor.empty((per,), abi.BF16)
        for i in range(args.layers):
            ops.fill_normal(src, 100 + i, 0.02)
            codes = abi.DeviceTensor.empty((per // 4 if code == 2 else per // 8,),
                                           abi.I32)
            scales = (abi.DeviceTensor.empty((2 * hid // 128 * (dim // 128),), abi.F32)
                      if code == 2 else
                      abi.DeviceTensor.empty((2 * hid * (dim // 32),), abi.F16))
            rc = lib().vx_b200_quantize(code, src.ptr, 2 * hid, dim, codes.ptr,
                                        scales.ptr)
            assert rc == 0
            quantised.append((codes, scales))
        run = lambda: [ops.nn_swiglu_quant(args.fmt, out, c, s, x, hid, dim)
                       for c, s in quantised]
        nbytes = (per + per // 16384 * 4 if code == 2 else per // 2 + per // 32 * 2) \
            + dim * 4 + hid * 4
    ms = _timed(torch, torch.cuda.Stream(), run, args.iters) / args.layers
    return dict(kernel="rowdot swiglu 22016x4096 %s" % args.fmt, us=ms * 1e3,
                bytes=nbytes, gbs=nbytes / ms / 1e6)


def gemm(torch, args):
    n = args.n
    if args.fmt == "f32":
        ta, tb, tc = (abi.DeviceTensor.empty((n, n), abi.F32) for _ in range(3))
        ops.fill_uniform(ta, 3, -1.0, 1.0)
        ops.fill_uniform(tb, 1003, -1.0, 1.0)
        ms = _timed(torch, torch.cuda.Stream(),
                    lambda: ops.matmul_into(tc, ta, tb), args.iters)
        return dict(kernel="f32 gemm %d^3 (three bf16 terms per value on tcgen05 "
                           "unless VXB_F32_TENSOR=0)" % n, us=ms * 1e3,
                    tflops=2.0 * n ** 3 / ms / 1e9, status=ops.kernel_status())
    if args.fmt in ("q4", "fp8"):
        # n positions against the 7B gate/up matrix in Q4_0 or fp8
        rows, cols = 22016, 4096
        src = abi.DeviceTensor.empty((rows * cols,), abi.BF16)
        ops.fill_normal(src, 100, 0.02)
        if args.fmt == "q4":
            codes = abi.DeviceTensor.empty((rows * cols // 8,), abi.I32)
            scales = abi.DeviceTensor.empty((rows * (cols // 32),), abi.F16)
            product = ops.gemm_q4
        else:
            codes = abi.DeviceTensor.empty((rows * cols // 4,), abi.I32)
            scales = abi.DeviceTensor.empty((rows // 128 * (cols // 128),), abi.F32)
            product = ops.gemm_fp8
        assert lib().vx_b200_quantize(3 if args.fmt == "q4" else 2, src.ptr, rows, cols,
                                      codes.ptr, scales.ptr) == 0
        x = abi.DeviceTensor.empty((n, cols), abi.F32)
        ops.fill_normal(x, 8, 1.0)
        y = abi.DeviceTensor.empty((n, rows), abi.F32)
        ms = _timed(torch, torch.cuda.Stream(),
                    lambda: product(y, codes, scales, x, n, rows, cols), args.iters)
        return dict(kernel="%s gemm: %d positions x (22016 x 4096), mma.sync with the "
                           "codes unpacked in registers" % (args.fmt, n), us=ms * 1e3,
                    tflops=2.0 * n * rows * cols / ms / 1e9, status=ops.kernel_status())
    ta, tb, tc = (abi.DeviceTensor.empty((n, n), abi.BF16) for _ in range(3))
    ops.fill_uniform(ta, 3, -1.0, 1.0)
    ops.fill_uniform(tb, 1003, -1.0, 1.0)
    ms = _timed(torch, torch.cuda.Stream(),
                lambda: ops.matmul_into(tc, ta, tb), args.iters)
    return dict(kernel="tcgen05 gemm bf16 %d^3" % n, us=ms * 1e3,
                tflops=2.0 * n ** 3 / ms / 1e9, status=ops.kernel_status())


def flash(torch, args):
    B, H, S, D = args.batch, args.heads, args.seq, 128
    ts = [abi.DeviceTensor.empty((B, H, S, D), abi.BF16) for _ in range(4)]
    for t, seed in zip(ts[:3], (10, 11, 12)):
        ops.fill_normal(t, seed, 1.0)
    scale = 1.0 / np.sqrt(D)
    ms = _timed(torch, torch.cuda.Stream(),
                lambda: ops.flash_attention(ts[0], ts[1], ts[2], ts[3], scale,
                                            True), args.iters)
    flops = 4.0 * B * H * D * S * (S + 1) / 2
    return dict(kernel="flash fwd causal [%d,%d,%d,%d]" % (B, H, S, D),
                us=ms * 1e3, tflops=flops / ms / 1e9, status=ops.kernel_status())


def attn(torch, args):
    qh = kvh = 32
    hd, pos, max_seq = 128, args.pos, 1024
    q = abi.DeviceTensor.empty((qh, hd), abi.F32)
    out = abi.DeviceTensor.empty((qh, hd), abi.F32)
    caches = []
    for i in range(8):                      # 8 layers' caches: 268 MB
        k = abi.DeviceTensor.empty((max_seq, kvh, hd), abi.F32)
        v = abi.DeviceTensor.empty((max_seq, kvh, hd), abi.F32)
        ops.fill_normal(k, 200 + i, 1.0)
        ops.fill_normal(v, 300 + i, 1.0)
        caches.append((k, v))
    ops.fill_normal(q, 98, 1.0)
    part = abi.DeviceTensor.empty(
        ops.nn_attention_scratch_shape(max_seq, qh, kvh, hd), abi.F32)
    ms = _timed(torch, torch.cuda.Stream(),
                lambda: [ops.nn_attention(out, part, q, k, v, pos, qh, kvh, hd)
                         for k, v in caches], args.iters) / len(caches)
    nbytes = 2 * (pos + 1) * kvh * hd * 4
    return dict(kernel="decode attention 32x128 at pos %d" % pos, us=ms * 1e3,
                bytes=nbytes, gbs=nbytes / ms / 1e6)


def decode16(torch, args):
    """A few layers of the 7B shape decoding `--batch` (8 or 16) sequences per
    step after `--pos` prompt positions: the tensor-core projections
    (rowdot_mma_kernel), attention and their small companions, for profiling."""
    from vx_b200 import llama
    shape = dict(llama.LLAMA2_7B)
    shape["n_layers"] = args.layers
    batch = args.batch if args.batch in (8, 16) else 16
    dec, tensors = llama.nn_bf16_model(max_seq=1024, batch=batch, **shape)
    rng = np.random.default_rng(1)
    for _ in range(args.pos):
        dec.step([int(t) for t in rng.integers(0, shape["vocab"], batch)],
                 fetch=False)
    ms = _timed(torch, torch.cuda.ExternalStream(dec.stream),
                lambda: dec.step(None, fetch=False), args.iters)
    dec.close()
    return dict(kernel="decode step, %d layers of the 7B shape, %d sequences, "
                       "position %d" % (args.layers, batch, args.pos),
                us=ms * 1e3, status=ops.kernel_status())


def shard(torch, args):
    """One rank's share of the 7B shape at tensor-parallel degree `--ranks`, run
    alone on one GPU (no exchange): heads, MLP rows and vocabulary divided by
    the ranks, the width kept. The decode step at position `--pos`: what a
    rank's chain of kernels costs apart from the exchange."""
    from vx_b200 import llama
    r = args.ranks
    shape = dict(dim=4096, hidden=11008 // r, n_layers=32, q_heads=32 // r,
                 kv_heads=32 // r, head_dim=128, vocab=32000 // r)
    dec, tensors = llama.nn_bf16_model(max_seq=1024, batch=1, **shape)
    rng = np.random.default_rng(1)
    for t in rng.integers(0, shape["vocab"], args.pos):
        dec.step([int(t)], fetch=False)
    ms = _timed(torch, torch.cuda.ExternalStream(dec.stream),
                lambda: dec.step(None, fetch=False), max(args.iters, 20))
    phases = None
    trace = dec.step_trace()      # with VXB_STEP_TRACE=1 and the one-launch step
    if trace is not None:
        t = trace.astype(np.int64)
        layers = t[:-1].reshape(32, 4, 6)[4:]          # skip the first layers
        names = ["qkv", "wo", "gate_up", "down"]
        phases = {}
        for k, name in enumerate(names):
            o = layers[:, k]
            phases[name] = dict(barrier=float((o[:, 1] - o[:, 0]).mean()) / 1e3,
                                stage_x=float((o[:, 2] - o[:, 1]).mean()) / 1e3,
                                rows=float((o[:, 3] - o[:, 2]).mean()) / 1e3)
        q = layers[:, 0]
        phases["attention"] = dict(barrier=float((q[:, 4] - q[:, 3]).mean()) / 1e3,
                                   units=float((q[:, 5] - q[:, 4]).mean()) / 1e3)
        phases["layer"] = float((layers[1:, 0, 0] - layers[:-1, 0, 0]).mean()) / 1e3
        phases["logits"] = dict(barrier=float(t[-1, 1] - t[-1, 0]) / 1e3,
                                stage_x=float(t[-1, 2] - t[-1, 1]) / 1e3,
                                rows=float(t[-1, 3] - t[-1, 2]) / 1e3)
    per_step = dec.kernels_per_step
    dec.close()
    nbytes = llama.weight_bytes_per_token(**shape)
    return dict(kernel="decode step of 1/%d of the 7B shape, position %d" % (r, args.pos),
                us=ms * 1e3, us_per_layer=ms * 1e3 / 32, tokens_per_s=1e3 / ms,
                weight_gbs=nbytes / ms / 1e6, status=ops.kernel_status(),
                kernels_per_step=per_step,
                phases_us_seen_by_block_0=phases)


def prefill(torch, args):
    """A 512-token prompt through `--layers` layers of the 7B shape in one pass
    (vx_decoder_prefill): the multi-position GEMMs, their finishing kernels and
    the f32 attention over the prompt."""
    import time
    from vx_b200 import llama
    shape = dict(llama.LLAMA2_7B)
    shape["n_layers"] = args.layers
    if args.fmt in ("q4", "fp8"):
        dec, tensors = llama.nn_quant_model(args.fmt, max_seq=1024, **shape)
    else:
        dec, tensors = llama.nn_bf16_model(max_seq=1024, batch=1, **shape)
    prompt = np.random.default_rng(8).integers(0, shape["vocab"], 512)
    best = None
    for _ in range(max(2, args.iters)):
        dec.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dec.prefill(prompt)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        best = ms if best is None else min(best, ms)
    dec.close()
    return dict(kernel="prefill of 512 tokens, %d layers of the 7B shape, %s weights"
                       % (args.layers, args.fmt), ms=best, ms_per_layer=best / args.layers, status=ops.kernel_status())


def moe(torch, args):
    """The experts of a mixture-of-experts layer for --n positions: 8 experts of
    14336 x 4096 in Q4_0, 2 a position. The router, the grouping by expert, and
    the two expert projections: grouped on the tensor cores, and position by
    position through the one-position kernels."""
    experts, k, dim, inter, n = 8, 2, 4096, 14336, args.n
    logits = abi.DeviceTensor.empty((n, experts), abi.F32)
    ops.fill_normal(logits, 7, 1.0)
    ids = abi.DeviceTensor.empty((n, k), abi.I32)
    wts = abi.DeviceTensor.empty((n, k), abi.F32)
    x = abi.DeviceTensor.empty((n, dim), abi.F32)
    ops.fill_normal(x, 8, 1.0)
    y = abi.DeviceTensor.empty((n, dim), abi.F32)
    ops.fill_normal(y, 9, 1.0)

    def q4_experts(rows, cols, seed):
        codes = abi.DeviceTensor.empty((experts * rows * cols // 8,), abi.I32)
        scales = abi.DeviceTensor.empty((experts * rows * (cols // 32),), abi.F16)
        src = abi.DeviceTensor.empty((rows * cols,), abi.BF16)
        for e in range(experts):
            ops.fill_normal(src, seed + e, 0.02)
            rc = lib().vx_b200_quantize(
                3, src.ptr, rows, cols, codes.ptr + e * rows * cols // 2,
                scales.ptr + e * rows * (cols // 32) * 2)
            assert rc == 0
        src.free()
        return codes, scales
    gu, gu_s = q4_experts(2 * inter, dim, 100)
    dn, dn_s = q4_experts(dim, inter, 200)
    pairs = n * k
    blocks = (pairs + 255) // 256
    counts = abi.DeviceTensor.empty((blocks, experts), abi.I32)
    base = abi.DeviceTensor.empty((blocks, experts), abi.I32)
    starts = abi.DeviceTensor.empty((experts + 1,), abi.I32)
    mid = abi.DeviceTensor.empty((pairs, inter), abi.F32)
    mid_rows = abi.DeviceTensor.empty((pairs, inter), abi.F32)
    scratch = abi.DeviceTensor.empty((pairs, dim), abi.F32)
    flat = ids.view(0, (pairs,))
    stream = torch.cuda.Stream()
    t_router = _timed(torch, stream,
                      lambda: ops.nn_top_k_rows(ids, wts, logits, n, experts, k), args.iters)
    grouped = {}
    for align in (8, 16):
        room = pairs + experts * (align - 1)
        order = abi.DeviceTensor.empty((room,), abi.I32)
        tile_expert = abi.DeviceTensor.empty(((room + align - 1) // align,), abi.I32)
        t_group = _timed(torch, stream,
                         lambda: ops.nn_moe_group(order, counts, base, starts, tile_expert,
                                                  flat, experts, align), args.iters)
        t_up = _timed(torch, stream,
                      lambda: ops.moe_swiglu_q4_grouped(mid, gu, gu_s, order, tile_expert,
                                                        align, x, n, k, inter, dim,
                                                        experts), args.iters)
        t_down = _timed(torch, stream,
                        lambda: ops.moe_down_q4_add_grouped(
                            y, dn, dn_s, order, tile_expert, align, wts.view(0, (pairs,)),
                            mid, scratch, n, k, dim, inter, experts), args.iters)
        grouped[align] = (t_group, t_up, t_down)
        order.free()
        tile_expert.free()
    t_group, t_up, t_down = grouped[16]
    t_up_rows = _timed(torch, stream,
                       lambda: ops.nn_moe_swiglu_q4_rows(mid_rows, gu, gu_s, ids, x, n, k,
                                                         inter, dim, experts), 1)
    t_down_rows = _timed(torch, stream,
                         lambda: ops.nn_moe_down_q4_add_rows(y, dn, dn_s, ids, wts,
                                                             mid_rows, n, k, dim, inter,
                                                             experts), 1)
    a, b = mid.to_host(), mid_rows.to_host()
    status = ops.kernel_status()
    for held in (logits, ids, wts, x, y, gu, gu_s, dn, dn_s, counts, base, starts, mid,
                 mid_rows, scratch):
        held.free()
    flop = 2.0 * pairs * 3 * inter * dim
    weight_bytes = experts * 3 * inter * dim * (0.5 + 2.0 / 32)
    return dict(kernel="experts of %d positions: 8 x (14336 x 4096) Q4_0, 2 a position" % n,
                router_us=t_router * 1e3, group_us=t_group * 1e3,
                swiglu_grouped_ms=t_up, down_grouped_ms=t_down,
                swiglu_grouped_align8_ms=grouped[8][1], down_grouped_align8_ms=grouped[8][2],
                swiglu_rows_ms=t_up_rows, down_rows_ms=t_down_rows,
                grouped_tflops=flop / ((t_up + t_down) * 1e-3) / 1e12,
                weights_gb=weight_bytes / 1e9,
                grouped_vs_rows_max_rel=float(np.abs(a - b).max() / np.abs(b).max()),
                status=status)


def main():
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["rowdot", "gemm", "flash", "attn", "decode16",
                                     "shard", "prefill", "moe"])
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--fmt", default="bf16", choices=["bf16", "fp8", "q4", "f32"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--pos", type=int, default=600)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    print(json.dumps(dict(rowdot=rowdot, gemm=gemm, flash=flash, attn=attn,
                          decode16=decode16, shard=shard,
                          prefill=prefill, moe=moe)[args.case](torch, args)))


if __name__ == "__main__":
    main()
