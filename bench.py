"""Benchmark of the GPU execution path behind Vx's tensor operators.

Headline (the JSON line's metric/value): greedy decode of a Llama-2-7B-shaped
bf16 model, batch 1, through the whole-token entry point -- tokens/s after a
512-token prompt, tensor-parallel over --gpus ranks of one box.  A "step" is
one decoded token.  The same line carries the bf16 GEMM and flash-attention
figures of the other configurations (N=1 only), the roofline of the dominant
kernel, and the CPU baseline.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT = 512
MAX_SEQ = 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0,
                source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,"
              "clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index),
                 "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)),
                    reasons=sorted(reasons), samples=len(sm))


# ---- the CPU arm -----------------------------------------------------------------
def cpu_decode_baseline(threads):
    """The oracle's std::nn decode step at Llama-2-7B shapes on the host cores.
    A bounded sample: one full layer (all five operators) at position 512 plus
    the classifier, timed, and scaled to 32 layers."""
    from oracle import vx_oracle as oracle
    from vx_b200 import llama
    oracle.set_threads(threads)
    s = llama.LLAMA2_7B
    dim, hid, hd, qh, kvh = s["dim"], s["hidden"], s["head_dim"], s["q_heads"], s["kv_heads"]
    pos = PROMPT
    rng = np.random.default_rng(7)

    def w16(n):
        return rng.integers(0x3000, 0x3C00, n, dtype=np.uint16)  # small positive bf16

    wqkv, bq = w16((qh + 2 * kvh) * hd * dim), np.zeros((qh + 2 * kvh) * hd, np.uint16)
    wo, wgu, wd = w16(dim * dim), w16(2 * hid * dim), w16(dim * hid)
    norm = w16(dim)
    head = w16(s["vocab"] * dim)
    x = rng.standard_normal(dim).astype(np.float32)
    kc = rng.standard_normal((pos + 1, kvh, hd)).astype(np.float32)
    vc = rng.standard_normal((pos + 1, kvh, hd)).astype(np.float32)
    cos, sin = oracle.rope_tables(pos + 1, hd, 10000.0)

    def layer():
        xb = oracle.nn_rms_norm(x, norm, dim, 1e-5)
        q, k, v = oracle.nn_qkv(wqkv, bq, xb, qh, kvh, hd, dim)
        qr = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, pos)
        att = oracle.nn_attention(qr, kc, vc, pos)
        y = oracle.nn_matvec(wo, att.reshape(-1), dim, dim, y=x)
        xb = oracle.nn_rms_norm(y, norm, dim, 1e-5)
        h = oracle.nn_swiglu(wgu, xb, hid, dim)
        return oracle.nn_matvec(wd, h, dim, hid, y=y)

    layer()
    t0 = time.perf_counter()
    reps = 3
    for _ in range(reps):
        layer()
    t_layer = (time.perf_counter() - t0) / reps
    t0 = time.perf_counter()
    oracle.nn_matvec(head, x, s["vocab"], dim)
    t_head = time.perf_counter() - t0
    per_token = t_layer * s["n_layers"] + t_head
    return dict(value=1.0 / per_token, unit="tokens/s", cores=threads,
                kind="port",
                sample="1 of 32 layers at position %d (mean of %d runs) + the "
                       "classifier, scaled to 32 layers: %.1f ms/layer, %.1f ms "
                       "classifier" % (pos, reps, t_layer * 1e3, t_head * 1e3))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    runs = []
    for _ in range(max(1, min(args.steps, 3))):
        runs.append(cpu_decode_baseline(threads))
    best = max(runs, key=lambda r: r["value"])
    line = dict(metric="llama2_7b_decode_tokens_per_s", value=best["value"],
                unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 / best["value"],
                higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16 weights, f32 accumulate", data="synthetic",
                impl="reference", config=workload_config(1, args.gpus),
                cpu_baseline=best,
                e2e=dict(value=best["value"], unit="tokens/s",
                         h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def workload_config(batch, gpus):
    return dict(workload="Llama-2-7B-shaped bf16 decoder (dim 4096, 32 layers, "
                         "32 heads x 128, FFN 11008, vocab 32000), greedy "
                         "decode after a %d-token random prompt" % PROMPT,
                batch=batch, prompt_tokens=PROMPT, max_seq=MAX_SEQ,
                parallelism="tp%d" % gpus,
                l2_policy="each step streams 13.2 GB of weights, far beyond "
                          "the 126 MB L2")


# ---- the GPU arm -------------------------------------------------------------------
def event_ms(torch, stream, fn):
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record(stream)
    fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop)


def bench_gemm(torch, peaks, n=8192, iters=20):
    """bf16 n^3 through the dispatch entry point, device-resident operands."""
    from vx_b200 import abi, ops
    from vx_b200.lib import lib
    ta, tb, tc = (abi.DeviceTensor.empty((n, n), abi.BF16) for _ in range(3))
    ops.fill_uniform(ta, 3, -1.0, 1.0)
    ops.fill_uniform(tb, 1003, -1.0, 1.0)
    stream = torch.cuda.Stream()
    lib().vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    try:
        for _ in range(3):
            ops.matmul_into(tc, ta, tb)
        stream.synchronize()
        ms = event_ms(torch, stream, lambda: [ops.matmul_into(tc, ta, tb)
                                              for _ in range(iters)]) / iters
        status = ops.kernel_status()
    finally:
        lib().vx_cuda_set_stream(None)
    for t in (ta, tb, tc):
        t.free()
    tflops = 2.0 * n ** 3 / ms / 1e9
    return dict(workload="bf16 %d^3, f32 accumulate, bf16 out" % n,
                tflops=tflops, ms=ms, frac_of_measured_cublas=tflops / peaks["bf16_tflops"],
                frac_of_nominal_2250=tflops / 2250.0, kernel_status=status,
                iters=iters)


def bench_flash(torch, peaks, B=8, H=32, S=4096, D=128, iters=5):
    from vx_b200 import abi, ops
    from vx_b200.lib import lib
    ts = [abi.DeviceTensor.empty((B, H, S, D), abi.BF16) for _ in range(4)]
    for t, seed in zip(ts[:3], (10, 11, 12)):
        ops.fill_normal(t, seed, 1.0)
    stream = torch.cuda.Stream()
    lib().vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    scale = 1.0 / np.sqrt(D)
    try:
        for _ in range(2):
            ops.flash_attention(ts[0], ts[1], ts[2], ts[3], scale, True)
        stream.synchronize()
        ms = event_ms(torch, stream, lambda: [
            ops.flash_attention(ts[0], ts[1], ts[2], ts[3], scale, True)
            for _ in range(iters)]) / iters
        status = ops.kernel_status()
    finally:
        lib().vx_cuda_set_stream(None)
    for t in ts:
        t.free()
    flops = 4.0 * B * H * D * S * (S + 1) / 2
    tflops = flops / ms / 1e9
    return dict(workload="bf16 causal forward [%d,%d,%d,%d]" % (B, H, S, D),
                tflops=tflops, ms=ms, flops_counted="causal: 4*B*H*D*S*(S+1)/2",
                frac_of_measured_cublas=tflops / peaks["bf16_tflops"],
                kernel_status=status, iters=iters)


def bench_dominant_kernel(torch, tensors, peaks, shape, iters=3):
    """The gate/up projection + SwiGLU of every layer in turn (32 different
    180 MB matrices, so nothing is left in L2), timed with CUDA events on the
    stream it is launched on."""
    from vx_b200 import abi, ops
    from vx_b200.lib import lib
    dim, hid = shape["dim"], shape["hidden"]
    x = abi.DeviceTensor.empty((dim,), abi.F32)
    ops.fill_normal(x, 99, 1.0)
    out = abi.DeviceTensor.empty((hid,), abi.F32)
    ws = [abi.DeviceTensor(t.data_ptr(), (2 * hid * dim,), abi.BF16, abi.home_gpu())
          for t in tensors["w_gate"]]
    stream = torch.cuda.Stream()
    lib().vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    try:
        for w in ws[:3]:
            ops.nn_swiglu(out, w, x, hid, dim)
        stream.synchronize()
        launches = iters * len(ws)
        ms = event_ms(torch, stream, lambda: [ops.nn_swiglu(out, w, x, hid, dim)
                                              for _ in range(iters) for w in ws])
    finally:
        lib().vx_cuda_set_stream(None)
    per_launch_ms = ms / launches
    bytes_per_launch = 2 * hid * dim * 2 + dim * 4 + hid * 4
    achieved = bytes_per_launch / per_launch_ms / 1e6
    return dict(bound="hbm", kernel="rowdot_kernel<bf16, batch 1, SwiGLU> "
                                    "(gate/up projection of one layer)",
                achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                frac=achieved / peaks["hbm_gbs"], peak_source=peaks["source"],
                bytes_per_launch=bytes_per_launch, us_per_launch=per_launch_ms * 1e3,
                launches_timed=launches,
                # dram__bytes_read.sum of one launch under ncu (180 405 248 B) plus the
                # 44 KB it writes; the profiler's own save/restore writes are left out
                # (the capture is summarised under profiles/)
                traffic=180405248 + 4 * shape["hidden"],
                traffic_source="ncu capture of this kernel on 4 of these matrices")


def bench_decode_batch(torch, llama, shape, peaks, batch):
    """The same model with `batch` sequences decoded together (the second
    half of the 7B configuration): aggregate tokens/s after a 512-token prompt
    per sequence, argmax fed back on the GPU."""
    dec, tensors = llama.nn_bf16_model(max_seq=MAX_SEQ, batch=batch, **shape)
    stream = torch.cuda.ExternalStream(dec.stream)
    prompts = np.random.default_rng(8).integers(0, shape["vocab"], (batch, PROMPT))
    steps = 32
    try:
        for p in range(PROMPT):
            dec.step([int(t) for t in prompts[:, p]], fetch=False)
        for _ in range(4):
            dec.step(None, fetch=False)
        torch.cuda.synchronize()
        ms = event_ms(torch, stream,
                      lambda: [dec.step(None, fetch=False) for _ in range(steps)])
    finally:
        dec.close()
        del tensors
        torch.cuda.empty_cache()
    per_step_bytes = llama.weight_bytes_per_token(**shape)
    kv = 2 * shape["n_layers"] * shape["kv_heads"] * shape["head_dim"] * 4 * \
        (PROMPT + 4 + steps / 2.0 + 1) * batch
    gbs = (per_step_bytes + kv) / (ms / steps) / 1e6
    return dict(workload="same model, %d sequences per step" % batch,
                tokens_per_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps,
                steps=steps, hbm_gbs=gbs, frac_of_measured_hbm=gbs / peaks["hbm_gbs"])


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    from vx_b200 import abi
    abi.set_home_gpu(local)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from vx_b200 import collective, llama
    from vx_b200.lib import lib
    peaks = measured_peaks()
    shape = llama.LLAMA2_7B

    if multi:
        id_file = "/tmp/vx_nccl_id_%s" % os.environ.get("MASTER_PORT", "0")
        if rank == 0 and os.path.exists(id_file):
            os.remove(id_file)
        dist.barrier()
        os.environ["VX_NCCL_ID_FILE"] = id_file
        collective.join_job(rank, world)

    dec, tensors = llama.nn_bf16_model(max_seq=MAX_SEQ, batch=1, tp_rank=rank,
                                       tp_ranks=world, **shape)
    stream = torch.cuda.ExternalStream(dec.stream)
    prompt = np.random.default_rng(8).integers(0, shape["vocab"], PROMPT)

    def barrier():
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    def run_prompt():
        dec.reset()
        for t in prompt[:-1]:
            dec.step([int(t)], fetch=False)
        return dec.step([int(prompt[-1])])[0]

    # -- device-resident: the argmax feeds the next step on the GPU ------------
    run_prompt()
    for _ in range(args.warmup):
        dec.step(None, fetch=False)
    barrier()
    with ClockSampler(local) as clocks:
        ms = event_ms(torch, stream,
                      lambda: [dec.step(None, fetch=False) for _ in range(args.steps)])
        time.sleep(0.25)
    barrier()
    # -- end to end: a host token in, the argmax token out, every step ---------
    tok = run_prompt()
    for _ in range(args.warmup):
        tok = dec.step([tok])[0]
    barrier()
    holder = {"tok": tok}

    def e2e_steps():
        for _ in range(args.steps):
            holder["tok"] = dec.step([holder["tok"]])[0]
    e2e_ms = event_ms(torch, stream, e2e_steps)
    barrier()

    # -- the prompt itself: one decode step per token, and sixteen positions per
    #    pass (vx_decoder_prefill); one GPU only
    prefill = None
    if not multi and not args.no_extras:
        def timed_prompt(fn):
            dec.reset()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            tok = fn()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1e3, tok
        step_ms, tok_a = timed_prompt(run_prompt)
        rows_ms, tok_b = timed_prompt(lambda: dec.prefill(prompt))
        prefill = dict(prompt_tokens=PROMPT, one_step_per_token_ms=step_ms,
                       sixteen_positions_per_pass_ms=rows_ms,
                       tokens_per_s=PROMPT / (rows_ms / 1e3),
                       same_next_token=bool(tok_a == tok_b),
                       timing="host clock around the whole prompt, "
                              "synchronised on both sides")

    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if multi:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(v) for v in times.cpu())
    launches = dec.kernels_per_step * args.steps

    if rank == 0:
        tokens_per_s = args.steps / (ms / 1e3)
        per_token_bytes = llama.weight_bytes_per_token(**shape)
        mean_pos = PROMPT + args.warmup + args.steps / 2.0
        kv_bytes = 2 * shape["n_layers"] * shape["kv_heads"] * shape["head_dim"] * 4 * (mean_pos + 1)
        step_gbs = (per_token_bytes + kv_bytes) / world / (ms / args.steps) / 1e6
        line = dict(
            metric="llama2_7b_decode_tokens_per_s", value=tokens_per_s,
            unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
            ms_per_step=ms / args.steps, higher_is_better=True,
            scaling="strong", vs_baseline=None,
            dtype="bf16 weights, f32 activations and accumulate",
            data="synthetic", config=workload_config(1, world),
            e2e=dict(value=args.steps / (e2e_ms / 1e3), unit="tokens/s",
                     h2d_bytes_per_step=4, d2h_bytes_per_step=4),
            gpu_launches=launches, kernels_per_step=dec.kernels_per_step,
            clocks=clocks.summary(),
            step_roofline=dict(
                bound="hbm", bytes_per_step_per_gpu=(per_token_bytes + kv_bytes) / world,
                achieved=step_gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                frac=step_gbs / peaks["hbm_gbs"], peak_source=peaks["source"]))
        if not multi:
            line["roofline"] = bench_dominant_kernel(torch, tensors, peaks, shape)
        if prefill:
            line["prefill"] = prefill
    dec.close()
    del tensors
    torch.cuda.empty_cache()

    if rank == 0 and not multi and not args.no_extras:
        try:
            line["decode_batch16"] = bench_decode_batch(torch, llama, shape, peaks, 16)
            # attention before the GEMMs: seconds of dense GEMM leave the GPU at
            # its power cap, and what runs next is measured at lower clocks
            line["flash_attention"] = bench_flash(torch, peaks)
            line["gemm"] = bench_gemm(torch, peaks)
            # the other sizes of the GEMM configuration (2048 fits L2: noted)
            line["gemm_sweep"] = {
                str(n): round(bench_gemm(torch, peaks, n=n, iters=it)["tflops"], 1)
                for n, it in ((2048, 50), (4096, 30), (16384, 5))}
        except RuntimeError as e:        # reported, never hidden
            line["extras_error"] = str(e)
    if rank == 0:
        if not multi:
            line["cpu_baseline"] = cpu_decode_baseline(os.cpu_count() or 1)
        print(json.dumps(line))
    if multi:
        collective.leave_job()
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the GEMM and flash-attention figures")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
