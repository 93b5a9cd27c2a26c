"""Benchmark of the GPU execution path behind Vx's tensor operators.

Headline (the JSON line's metric/value): greedy decode of a Llama-2-7B-shaped
bf16 model, batch 1, through the whole-token entry point -- tokens/s after a
512-token prompt, tensor-parallel over --gpus ranks of one box.  A "step" is
one decoded token.  The same line carries, at every N, a digest of the tokens
the model generates from a fixed prompt (so that every tensor-parallel degree
shows the tokens of one GPU), and at N=1 the figures of the other
configurations (f32 1024^3, the bf16 GEMM sweep, flash attention, 16
sequences per step), each with its error against the CPU oracle on sampled
rows, the roofline of the dominant kernel, and the CPU baseline.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import ctypes as C
import hashlib
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
MAX_SEQ = 4096                   # the configuration's context length
DIGEST_PROMPT, DIGEST_STEPS = 16, 64
CPU_CHECK_STEPS = 8              # oracle steps compared with the GPU's tokens
CPU_TIMED_STEPS = 8              # oracle steps timed at positions >= 512


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
                 "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 2.0     # the first sample takes a moment
            while not self.lines and time.time() < deadline:
                time.sleep(0.01)
            self.lines.clear()               # what follows is under load
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


def digest_prompt(vocab):
    return [int(t) for t in np.random.default_rng(8).integers(0, vocab, PROMPT)
            [:DIGEST_PROMPT]]


def tokens_sha(tokens):
    return hashlib.sha256(np.asarray(tokens, np.int32).tobytes()).hexdigest()[:16]


# ---- the CPU arm -----------------------------------------------------------------
def random_kv_rows(kc, vc, first, last, seed=5):
    """Rows first..last-1 of every layer's cache get N(0,1) values: the rows a
    512-token prompt would have left (their values do not change the time)."""
    rng = np.random.default_rng(seed)
    for l in range(kc.shape[0]):
        kc[l, first:last] = rng.standard_normal(kc[l, first:last].shape,
                                                dtype=np.float32)
        vc[l, first:last] = rng.standard_normal(vc[l, first:last].shape,
                                                dtype=np.float32)


def cpu_timed_steps(oracle, hm, kv, first_pos, steps):
    """Whole decode steps of the oracle (all 32 layers + classifier + argmax)
    at positions first_pos, first_pos + 1, ...: seconds per step, each."""
    cfg, (kc, vc) = hm["cfg"], kv
    tok, times = 1, []
    for i in range(steps):
        t0 = time.perf_counter()
        tok = oracle.nn_decode_step(cfg, hm["embed"], hm["layers"],
                                    hm["final_norm"], hm["lm_head"], hm["cos"],
                                    hm["sin"], kc, vc, tok, first_pos + i)
        times.append(time.perf_counter() - t0)
    return times


def synthetic_host_model(oracle, shape, max_seq):
    """A 7B-shaped model for the CPU arm alone (no GPU involved): one layer of
    random bf16 weights, laid down 32 times (32 distinct 400 MB blocks of
    memory with the same contents: the time of a step does not depend on the
    values, only on streaming 13 GB)."""
    from vx_b200 import llama
    cfg = oracle.NnConfig(shape["dim"], shape["hidden"], shape["n_layers"],
                          shape["q_heads"], shape["kv_heads"], shape["head_dim"],
                          shape["vocab"], max_seq, 1e-5, 10000.0)
    per_layer = oracle.nn_layer_params(cfg)
    rng = np.random.default_rng(7)
    one = oracle.f32_to_bf16(rng.standard_normal(per_layer, dtype=np.float32)
                             * np.float32(0.02))
    layers = np.tile(one, shape["n_layers"])
    table = oracle.f32_to_bf16(
        rng.standard_normal(shape["vocab"] * shape["dim"], dtype=np.float32)
        * np.float32(0.02))
    cos, sin = llama.rope_tables(max_seq, shape["head_dim"], 10000.0)
    ones = oracle.f32_to_bf16(np.ones(shape["dim"], np.float32))
    return dict(cfg=cfg, layers=layers, embed=table, final_norm=ones,
                lm_head=table, cos=cos, sin=sin)


def run_reference(args):
    """The reference's CPU path (its port: the reference itself needs Rust and
    LLVM to build) on all host cores: K whole decode steps of the 7B-shaped
    model at positions 512.., after W untimed ones."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import vx_oracle as oracle
    from vx_b200 import llama
    threads = os.cpu_count() or 1
    oracle.set_threads(threads)
    shape = llama.LLAMA2_7B
    max_seq = PROMPT + args.warmup + args.steps + 8
    hm = synthetic_host_model(oracle, shape, max_seq)
    kv_shape = (shape["n_layers"], max_seq, shape["kv_heads"], shape["head_dim"])
    kv = (np.zeros(kv_shape, np.float32), np.zeros(kv_shape, np.float32))
    random_kv_rows(kv[0], kv[1], 0, PROMPT)
    cpu_timed_steps(oracle, hm, kv, PROMPT, args.warmup)
    times = cpu_timed_steps(oracle, hm, kv, PROMPT + args.warmup, args.steps)
    total = float(sum(times))
    value = args.steps / total
    base = dict(value=value, unit="tokens/s", cores=threads, kind="port",
                sample="%d whole decode steps (32 layers, classifier, argmax) "
                       "at positions %d..%d after %d untimed ones; KV rows "
                       "below 512 random" % (args.steps, PROMPT + args.warmup,
                                             PROMPT + args.warmup + args.steps - 1,
                                             args.warmup))
    line = dict(metric="llama2_7b_decode_tokens_per_s", value=value,
                unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * total / args.steps,
                higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16 weights, f32 activations and accumulate",
                data="synthetic", impl="reference",
                config=workload_config(1, args.gpus), cpu_baseline=base,
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0,
                         d2h_bytes_per_step=0))
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


class on_stream:
    """The library's work goes to `stream` inside the block."""

    def __init__(self, stream):
        self.stream = stream

    def __enter__(self):
        from vx_b200.lib import lib
        lib().vx_cuda_set_stream(C.c_void_p(self.stream.cuda_stream))

    def __exit__(self, *exc):
        from vx_b200.lib import lib
        lib().vx_cuda_set_stream(None)


def bench_small_llama(torch, oracle, llama):
    """Configuration 2: the f32 program's small decoder (dim 288, 6 layers, 6
    heads, hidden 768, vocab 32000, seq 256, N(0, 0.02^2) from seed 42), 100
    greedy tokens from BOS = 1 with the argmax fed back on the GPU; the CPU
    program on one thread (the reference's own way) beside it, and the tokens
    compared. 60 MB of weights sit in L2: a latency figure, not a bandwidth
    one."""
    flat, offsets = llama.small_f32_weights()
    cfg = oracle.LlamaConfig(288, 768, 6, 6, 6, 32000, 256)
    oracle.set_threads(1)
    t0 = time.perf_counter()
    want = list(oracle.llama_generate(cfg, flat, 1, 100))
    cpu_s = time.perf_counter() - t0
    oracle.set_threads(os.cpu_count() or 1)
    dec = llama.small_f32_decoder(flat, offsets)
    stream = torch.cuda.ExternalStream(dec.stream)
    dec.step([1], fetch=False)
    for _ in range(99):
        dec.step(None, fetch=False)
    dec.reset()
    torch.cuda.synchronize()
    first = dec.step([1])[0]
    ms = event_ms(torch, stream,
                  lambda: [dec.step(None, fetch=False) for _ in range(98)])
    last = dec.step(None)[0]
    dec.reset()
    got, tok = [1], dec.step([1])[0]
    got.append(tok)
    for _ in range(99):
        tok = dec.step(None)[0]
        got.append(tok)
    dec.close()
    return dict(workload="f32 decoder dim 288, 6 layers, vocab 32000, 100 greedy "
                         "tokens from BOS", tokens_per_s=98 / (ms / 1e3),
                us_per_token=ms * 1e3 / 98, tokens_equal_cpu=bool(got == want),
                cpu_one_thread_tokens_per_s=100 / cpu_s,
                consistent=bool(first == want[1] and last == want[100]))


def bench_gemm_f32(torch, oracle, n=1024, iters=50):
    """Configuration 1: f32 n^3 with A, B uniform[-1,1) from seeds 0 and 1,
    through the dispatch entry point with device-resident operands and with
    host operands (staged both ways inside the call); the whole C against the
    CPU loop nest, which is also timed on one thread (the reference's host
    GEMM is one thread) and on all cores."""
    from vx_b200 import abi, ops
    a = np.random.default_rng(0).uniform(-1, 1, (n, n)).astype(np.float32)
    b = np.random.default_rng(1).uniform(-1, 1, (n, n)).astype(np.float32)
    ta, tb = abi.DeviceTensor.from_host(a), abi.DeviceTensor.from_host(b)
    tc = abi.DeviceTensor.empty((n, n), abi.F32)
    stream = torch.cuda.Stream()
    with on_stream(stream):
        for _ in range(3):
            ops.matmul_into(tc, ta, tb)
        stream.synchronize()
        ms = event_ms(torch, stream, lambda: [ops.matmul_into(tc, ta, tb)
                                              for _ in range(iters)]) / iters
    got = tc.to_host()
    # the same product on the FP32 pipe (the tensor-core route switched off)
    os.environ["VXB_F32_TENSOR"] = "0"
    try:
        with on_stream(stream):
            ops.matmul_into(tc, ta, tb)
            stream.synchronize()
            pipe_ms = event_ms(torch, stream, lambda: [ops.matmul_into(tc, ta, tb)
                                                       for _ in range(iters)]) / iters
        got_pipe = tc.to_host()
    finally:
        del os.environ["VXB_F32_TENSOR"]
    t0 = time.perf_counter()
    host = ops.matmul_host(a, b, slot=False)
    host_ms = (time.perf_counter() - t0) * 1e3
    threads = os.cpu_count() or 1
    oracle.set_threads(1)
    t0 = time.perf_counter()
    want = oracle.gemm(a, b)
    cpu1 = time.perf_counter() - t0
    oracle.set_threads(threads)
    t0 = time.perf_counter()
    oracle.gemm(a, b)
    cpun = time.perf_counter() - t0
    for t in (ta, tb, tc):
        t.free()
    flop = 2.0 * n ** 3
    return dict(workload="f32 %d^3, uniform[-1,1) seeds 0/1; f32 in and out, "
                         "on the tensor cores as three exact bf16 terms per value"
                         % n,
                tflops=flop / ms / 1e9, ms=ms, iters=iters,
                rel_frobenius_err=float(np.linalg.norm(got - want) /
                                        np.linalg.norm(want)),
                fp32_pipe_tflops=flop / pipe_ms / 1e9, fp32_pipe_ms=pipe_ms,
                fp32_pipe_rel_frobenius_err=float(np.linalg.norm(got_pipe - want) /
                                                  np.linalg.norm(want)),
                host_operands_ms=host_ms,
                host_operands_rel_err=float(np.linalg.norm(host - want) /
                                            np.linalg.norm(want)),
                cpu_one_thread_s=cpu1, cpu_all_cores_s=cpun, cpu_cores=threads,
                tolerance=1e-4)


def bench_gemm(torch, oracle, peaks, n=8192, iters=20, check_rows=8):
    """bf16 n^3 through the dispatch entry point, device-resident operands;
    `check_rows` sampled rows of C against the oracle's f32-accumulate loop."""
    from vx_b200 import abi, ops
    ta, tb, tc = (abi.DeviceTensor.empty((n, n), abi.BF16) for _ in range(3))
    ops.fill_uniform(ta, 3, -1.0, 1.0)
    ops.fill_uniform(tb, 1003, -1.0, 1.0)
    stream = torch.cuda.Stream()
    with on_stream(stream):
        for _ in range(3):
            ops.matmul_into(tc, ta, tb)
        stream.synchronize()
        # the way the measured cuBLAS peaks were taken: the best of ten single
        # products from a rested GPU (a burst, before the power cap bites: what
        # ran before this leg has left the chip at its cap, so it idles for a
        # moment first), and back to back
        time.sleep(1.5 if n >= 8192 else 0.0)
        burst_ms = min(event_ms(torch, stream, lambda: ops.matmul_into(tc, ta, tb))
                       for _ in range(10))
        ms = event_ms(torch, stream, lambda: [ops.matmul_into(tc, ta, tb)
                                              for _ in range(iters)]) / iters
        status = ops.kernel_status()
    out = dict(workload="bf16 %d^3, f32 accumulate, bf16 out" % n,
               tflops=2.0 * n ** 3 / burst_ms / 1e9, ms=burst_ms,
               timing="best of 10 single products, CUDA events (as the measured "
                      "cuBLAS burst figure was taken)",
               tflops_back_to_back=2.0 * n ** 3 / ms / 1e9, ms_back_to_back=ms,
               kernel_status=status, iters=iters)
    out["frac_of_measured_cublas"] = out["tflops"] / peaks["bf16_tflops"]
    out["frac_of_nominal_2250"] = out["tflops"] / 2250.0
    if peaks.get("bf16_tflops_sustained"):
        out["back_to_back_frac_of_measured_cublas_sustained"] = \
            out["tflops_back_to_back"] / peaks["bf16_tflops_sustained"]
    if check_rows:
        rows = (np.arange(check_rows, dtype=np.int64) * 7919 + 13) % n
        a16, b16, c16 = ta.to_host(), tb.to_host(), tc.to_host()
        t0 = time.perf_counter()
        want = oracle.bf16_to_f32(oracle.gemm_bf16_rows(a16, b16, rows))
        cpu_s = time.perf_counter() - t0
        got = oracle.bf16_to_f32(c16[rows])
        out["rel_err_sampled_rows"] = float(np.linalg.norm(got - want) /
                                            np.linalg.norm(want))
        out["rows_checked"] = int(check_rows)
        out["tolerance"] = 2e-2
        out["cpu_all_cores_s_extrapolated"] = cpu_s * n / check_rows
    for t in (ta, tb, tc):
        t.free()
    return out


def bench_flash(torch, oracle, peaks, B=8, H=32, S=4096, D=128, iters=5):
    """Configuration 3, and sampled rows of a few (batch, head) pairs against
    the oracle's f32 attention over the same bf16 inputs."""
    from vx_b200 import abi, ops
    ts = [abi.DeviceTensor.empty((B, H, S, D), abi.BF16) for _ in range(4)]
    for t, seed in zip(ts[:3], (10, 11, 12)):
        ops.fill_normal(t, seed, 1.0)
    stream = torch.cuda.Stream()
    scale = 1.0 / np.sqrt(D)
    with on_stream(stream):
        for _ in range(2):
            ops.flash_attention(ts[0], ts[1], ts[2], ts[3], scale, True)
        stream.synchronize()
        ms = event_ms(torch, stream, lambda: [
            ops.flash_attention(ts[0], ts[1], ts[2], ts[3], scale, True)
            for _ in range(iters)]) / iters
        status = ops.kernel_status()
    rows = np.unique(np.concatenate([np.arange(5, S, 509), [0, 127, 128, S - 1]]))
    worst, cpu_s = 0.0, 0.0
    pairs = [(0, 0), (B // 2, H // 3), (B - 1, H - 1)]
    for b, h in pairs:
        at = (b * H + h) * S * D
        q, k, v, o = (t.view(at, (S, D)).to_host() for t in ts)
        t0 = time.perf_counter()
        want = oracle.attention_rows(q, k, v, scale, True, rows)
        cpu_s += time.perf_counter() - t0
        worst = max(worst, float(np.abs(oracle.bf16_to_f32(o)[rows] - want).max()))
    for t in ts:
        t.free()
    flops = 4.0 * B * H * D * S * (S + 1) / 2
    tflops = flops / ms / 1e9
    return dict(workload="bf16 causal forward [%d,%d,%d,%d]" % (B, H, S, D),
                tflops=tflops, ms=ms, flops_counted="causal: 4*B*H*D*S*(S+1)/2",
                frac_of_measured_cublas=tflops / peaks["bf16_tflops"],
                frac_of_nominal_2250=tflops / 2250.0,
                target="0.60 of tensor peak; both denominators are given",
                kernel_status=status, iters=iters, max_abs_err=worst,
                rows_checked=int(rows.size) * len(pairs), tolerance=2e-2,
                # the sampled rows average S/2 keys like all rows do
                cpu_all_cores_s_extrapolated=cpu_s * B * H * S /
                (rows.size * len(pairs)))


def bench_dominant_kernel(torch, tensors, peaks, shape, iters=3):
    """The gate/up projection + SwiGLU of every layer in turn (32 different
    180 MB matrices, so nothing is left in L2), timed with CUDA events on the
    stream it is launched on."""
    from vx_b200 import abi, ops
    dim, hid = shape["dim"], shape["hidden"]
    x = abi.DeviceTensor.empty((dim,), abi.F32)
    ops.fill_normal(x, 99, 1.0)
    out = abi.DeviceTensor.empty((hid,), abi.F32)
    ws = [abi.DeviceTensor(t.data_ptr(), (2 * hid * dim,), abi.BF16, abi.home_gpu())
          for t in tensors["w_gate"]]
    stream = torch.cuda.Stream()
    with on_stream(stream):
        for w in ws[:3]:
            ops.nn_swiglu(out, w, x, hid, dim)
        stream.synchronize()
        launches = iters * len(ws)
        ms = event_ms(torch, stream, lambda: [ops.nn_swiglu(out, w, x, hid, dim)
                                              for _ in range(iters) for w in ws])
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


def bench_decode_quant(torch, llama, shape, peaks, quant):
    """The same model with every layer's projections in fp8 (half the bytes of
    bf16) or Q4_0 (a quarter): tokens/s after a 512-token prompt, and the rate
    over the bytes such a step has to read."""
    dec, tensors = llama.nn_quant_model(quant, max_seq=MAX_SEQ, **shape)
    stream = torch.cuda.ExternalStream(dec.stream)
    prompt = np.random.default_rng(8).integers(0, shape["vocab"], PROMPT)
    steps = 64
    prompt_ms = {}
    try:
        if quant in ("q4", "fp8"):
            # the prompt in one pass (the codes unpacked once for sixteen
            # positions, on the tensor cores) beside one decode step per token;
            # same first token?
            def timed_prompt(fn):
                dec.reset()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                tok = fn()
                torch.cuda.synchronize()
                return (time.perf_counter() - t0) * 1e3, tok

            def stepped():
                for t in prompt[:-1]:
                    dec.step([int(t)], fetch=False)
                return dec.step([int(prompt[-1])])[0]
            timed_prompt(lambda: dec.prefill(prompt))        # warm
            rows_ms, tok_rows = timed_prompt(lambda: dec.prefill(prompt))
            step_ms, tok_steps = timed_prompt(stepped)
            prompt_ms = dict(prefill_ms=rows_ms, one_step_per_token_ms=step_ms,
                             first_token_equal=bool(tok_rows == tok_steps))
            # the other route: codes unpacked in registers, mma.sync
            knob = "VXB_Q4_PREFILL" if quant == "q4" else "VXB_FP8_PREFILL"
            os.environ[knob] = "mma"
            try:
                timed_prompt(lambda: dec.prefill(prompt))
                mma_ms, tok_mma = timed_prompt(lambda: dec.prefill(prompt))
            finally:
                del os.environ[knob]
            prompt_ms.update(prefill_mma_sync_ms=mma_ms,
                             first_token_equal_mma_sync=bool(tok_mma == tok_steps))
            timed_prompt(lambda: dec.prefill(prompt))   # the cache as the default leaves it
        else:
            for t in prompt:
                dec.step([int(t)], fetch=False)
        for _ in range(4):
            dec.step(None, fetch=False)
        torch.cuda.synchronize()
        ms = event_ms(torch, stream,
                      lambda: [dec.step(None, fetch=False) for _ in range(steps)])
    finally:
        dec.close()
        del tensors
        torch.cuda.empty_cache()
    per_layer = ((shape["q_heads"] + 2 * shape["kv_heads"]) * shape["head_dim"]
                 * shape["dim"] + shape["dim"] * shape["q_heads"] * shape["head_dim"]
                 + 3 * shape["dim"] * shape["hidden"])
    # codes + scales (fp8: 4 bytes per 16384 weights; Q4_0: 2 bytes per 32)
    layer_bytes = per_layer * (1.0 + 4.0 / 16384 if quant == "fp8"
                               else 0.5 + 2.0 / 32)
    head_bytes = shape["vocab"] * shape["dim"] * 2
    kv = 2 * shape["n_layers"] * shape["kv_heads"] * shape["head_dim"] * 4 * \
        (PROMPT + 4 + steps / 2.0 + 1)
    total = shape["n_layers"] * layer_bytes + head_bytes + kv
    gbs = total / (ms / steps) / 1e6
    return dict(workload="same model, layer projections in %s, batch 1" % quant,
                tokens_per_s=steps / (ms / 1e3), ms_per_step=ms / steps,
                steps=steps, bytes_per_step=total, hbm_gbs=gbs,
                frac_of_measured_hbm=gbs / peaks["hbm_gbs"], **prompt_ms)


def bench_moe_experts(torch, positions=512):
    """A mixture-of-experts layer's experts for a prompt of `positions`: 8 Q4_0
    experts of 14336 x 4096, 2 a position; router, grouping by expert, and both
    projections grouped on the tensor cores, beside the position-by-position
    exports (the same case as `python microbench.py moe`)."""
    import argparse
    import microbench
    r = microbench.moe(torch, argparse.Namespace(n=positions, iters=3))
    torch.cuda.empty_cache()
    grouped = r["router_us"] / 1e3 + r["group_us"] / 1e3 + r["swiglu_grouped_ms"] + \
        r["down_grouped_ms"]
    return dict(workload=r["kernel"], layer_ms_grouped=grouped,
                layer_ms_position_by_position=r["swiglu_rows_ms"] + r["down_rows_ms"],
                router_us=r["router_us"], group_us=r["group_us"],
                swiglu_grouped_ms=r["swiglu_grouped_ms"],
                down_grouped_ms=r["down_grouped_ms"],
                useful_tflops=r["grouped_tflops"],
                grouped_vs_rows_max_rel=r["grouped_vs_rows_max_rel"],
                kernel_status=r["status"])


def bench_skinny_layers(torch, llama, rank, world, alone=False):
    """The per-layer cost that is not weight streaming: a model with the 7B
    width but almost no weights (one head per rank, 64 MLP rows per rank),
    32 layers. alone: the rank's share as a model of its own, no exchange; the
    difference is two exchanges per layer."""
    ranks = 1 if alone else world
    skinny = dict(dim=4096, hidden=64 * ranks, n_layers=32, q_heads=ranks,
                  kv_heads=ranks, head_dim=128, vocab=64 * ranks)
    dec, tensors = llama.nn_bf16_model(max_seq=64, batch=1,
                                       tp_rank=0 if alone else rank,
                                       tp_ranks=ranks, **skinny)
    stream = torch.cuda.ExternalStream(dec.stream)
    dec.step([1], fetch=False)
    for _ in range(8):
        dec.step(None, fetch=False)
    torch.cuda.synchronize()
    steps = 24
    ms = event_ms(torch, stream,
                  lambda: [dec.step(None, fetch=False) for _ in range(steps)])
    dec.close()
    del tensors
    return ms * 1e3 / steps / skinny["n_layers"]


def bench_column_split(torch, dist, rank, world, n=16384, iters=3):
    """Configuration 4's multi-GPU half: C = A B with B column-split over the
    ranks; every rank computes its column block, the blocks are all-gathered
    (vx_collective_all_gather_bf16's NCCL call) and interleaved into the
    row-major C, all inside the timed region. The local GEMM is also timed
    alone, so the line says what the gather and the interleave cost."""
    from vx_b200 import abi, ops
    from vx_b200.lib import check, lib
    nl = n // world
    ta = abi.DeviceTensor.empty((n, n), abi.BF16)
    tb = abi.DeviceTensor.empty((n, nl), abi.BF16)
    tcl = abi.DeviceTensor.empty((n, nl), abi.BF16)
    tg = abi.DeviceTensor.empty((world, n, nl), abi.BF16)
    tc = abi.DeviceTensor.empty((n, n), abi.BF16)
    ops.fill_uniform(ta, 3, -1.0, 1.0)
    ops.fill_uniform(tb, 2003 + rank, -1.0, 1.0)
    stream = torch.cuda.Stream()

    def whole():
        check(lib().vx_b200_gemm_column_split(abi.BF16, n, nl, n, ta.ptr, tb.ptr,
                                              tcl.ptr, tg.ptr, tc.ptr))

    def local():
        check(lib().vx_b200_gemm(abi.BF16, 0, n, nl, n, ta.ptr, n, tb.ptr, nl,
                                 tcl.ptr, nl, None))

    with on_stream(stream):
        whole()
        local()
        stream.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ms = event_ms(torch, stream, lambda: [whole() for _ in range(iters)]) / iters
        dist.barrier()
        torch.cuda.synchronize()
        local_ms = event_ms(torch, stream,
                            lambda: [local() for _ in range(iters)]) / iters
        status = ops.kernel_status()
    times = torch.tensor([ms, local_ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, local_ms = (float(v) for v in times.cpu())
    for t in (ta, tb, tcl, tg, tc):
        t.free()
    flop = 2.0 * n ** 3
    return dict(workload="bf16 %d^3, B column-split over %d ranks, all-gather "
                         "of C + interleave inside the timed region" % (n, world),
                ms=ms, tflops_aggregate=flop / ms / 1e9,
                tflops_per_gpu=flop / world / ms / 1e9, local_gemm_ms=local_ms,
                gather_and_interleave_share=(ms - local_ms) / ms,
                kernel_status=status, iters=iters)


def cpu_baseline_with_the_model(oracle, hm, got_tokens, threads):
    """The CPU arm on the model the GPU decoded: the first CPU_CHECK_STEPS
    tokens after the digest prompt must be the GPU's (the oracle as checker),
    then whole steps are timed at positions >= 512 over random KV rows."""
    oracle.set_threads(threads)
    cfg = hm["cfg"]
    max_seq = PROMPT + CPU_TIMED_STEPS + 8
    shape = (cfg.n_layers, max_seq, cfg.kv_heads, cfg.head_dim)
    kv = (np.zeros(shape, np.float32), np.zeros(shape, np.float32))
    hm = dict(hm, cos=hm["cos"][:max_seq], sin=hm["sin"][:max_seq])
    cfg.max_seq = max_seq
    want = oracle.nn_generate(hm, digest_prompt(cfg.vocab), CPU_CHECK_STEPS,
                              max_seq, kv=kv)
    random_kv_rows(kv[0], kv[1], DIGEST_PROMPT + CPU_CHECK_STEPS, PROMPT)
    times = cpu_timed_steps(oracle, hm, kv, PROMPT, 1 + CPU_TIMED_STEPS)[1:]
    value = len(times) / float(sum(times))
    return dict(value=value, unit="tokens/s", cores=threads, kind="port",
                sample="%d whole decode steps (32 layers, classifier, argmax) of "
                       "this model at positions %d..%d after one untimed; KV "
                       "rows below 512 random" % (len(times), PROMPT + 1,
                                                  PROMPT + len(times)),
                tokens_checked=CPU_CHECK_STEPS,
                tokens_match_gpu=bool(list(want) ==
                                      list(got_tokens[:CPU_CHECK_STEPS])))


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

    # -- device-resident: the argmax feeds the next step on the GPU. Exactly
    #    `steps` steps per measurement; a short region is measured several
    #    times (the median counts) so that the clock record has samples.
    run_prompt()
    for _ in range(args.warmup):
        dec.step(None, fetch=False)
    barrier()
    repeats = 1 if args.steps >= 400 else 5
    measured = []
    with ClockSampler(local) as clocks:
        for _ in range(repeats):
            measured.append(event_ms(
                torch, stream,
                lambda: [dec.step(None, fetch=False) for _ in range(args.steps)]))
            barrier()
        time.sleep(0.1)
    ms = float(np.median(measured))
    # -- end to end: a host token in, the argmax token out, every step ---------
    tok = run_prompt()
    for _ in range(args.warmup):
        tok = dec.step([tok])[0]
    barrier()
    holder = {"tok": tok}

    def e2e_steps():
        for _ in range(args.steps):
            holder["tok"] = dec.step([holder["tok"]])[0]
    e2e_ms = float(np.median([event_ms(torch, stream, e2e_steps)
                              for _ in range(repeats)]))
    barrier()

    # -- what the model says: the tokens after a fixed 16-token prompt, the
    #    same at every tensor-parallel degree
    dec.reset()
    tok = None
    for t in digest_prompt(shape["vocab"]):
        tok = dec.step([t])[0]
    said = []
    for _ in range(DIGEST_STEPS):
        said.append(tok)
        tok = dec.step(None)[0]

    # -- the prompt itself: one decode step per token, and many positions per
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
        timed_prompt(lambda: dec.prefill(prompt))            # warm
        rows_ms, tok_b = timed_prompt(lambda: dec.prefill(prompt))
        after = [tok_b]
        for _ in range(15):
            after.append(dec.step(None)[0])
        dec.reset()
        tok = run_prompt()
        after_steps = [tok]
        for _ in range(15):
            after_steps.append(dec.step(None)[0])
        per_layer = ((shape["q_heads"] + 2 * shape["kv_heads"]) * shape["head_dim"]
                     * shape["dim"] + shape["dim"] * shape["q_heads"]
                     * shape["head_dim"] + 3 * shape["dim"] * shape["hidden"])
        flop = 2.0 * per_layer * shape["n_layers"] * (PROMPT - 1)
        prefill = dict(prompt_tokens=PROMPT, one_step_per_token_ms=step_ms,
                       prefill_ms=rows_ms,
                       tokens_per_s=PROMPT / (rows_ms / 1e3),
                       # the projections of 511 positions (the last prompt token
                       # is a decode step); the tensor cores execute three times
                       # as much, one product per bf16 term of an f32 activation
                       tflops_algorithmic=flop / rows_ms / 1e9,
                       tflops_executed=3 * flop / rows_ms / 1e9,
                       executed_frac_of_measured_cublas=3 * flop / rows_ms / 1e9
                       / peaks["bf16_tflops"],
                       same_next_token=bool(tok_a == tok_b),
                       same_16_following_tokens=bool(after == after_steps),
                       timing="host clock around the whole prompt, "
                              "synchronised on both sides")

    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if multi:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(v) for v in times.cpu())
    launches = dec.kernels_per_step * args.steps
    from vx_b200 import ops
    status = ops.kernel_status()

    line = None
    if rank == 0:
        tokens_per_s = args.steps / (ms / 1e3)
        per_token_bytes = llama.weight_bytes_per_token(**shape)
        mean_pos = PROMPT + args.warmup + args.steps * repeats / 2.0
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
            timed_repeats=repeats, kernel_status=status,
            tokens_sha=tokens_sha(said), tokens_head=said[:8],
            tokens_of="%d greedy tokens after the first %d ids of the prompt"
                      % (DIGEST_STEPS, DIGEST_PROMPT),
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

    host_model = None
    if rank == 0 and not multi:
        from oracle import vx_oracle as oracle
        host_model = oracle.nn_model_from_tensors(tensors, shape, MAX_SEQ)
    del tensors
    torch.cuda.empty_cache()

    try:
        line_extra = {}
        line_extra["skinny_us_per_layer"] = bench_skinny_layers(torch, llama, rank,
                                                                world)
        if multi:
            # the same share of the skinny model run alone on this GPU: what is
            # left is the exchange, twice per layer
            alone = bench_skinny_layers(torch, llama, rank, world, alone=True)
            line_extra["skinny_alone_us_per_layer"] = alone
            line_extra["exchange_us"] = (line_extra["skinny_us_per_layer"] - alone) / 2.0
        if multi and not args.no_extras:
            line_extra["gemm_column_split"] = bench_column_split(torch, dist, rank,
                                                                 world)
        if rank == 0:
            line.update(line_extra)
    except RuntimeError as e:            # reported, never hidden
        if rank == 0:
            line["extras_error"] = str(e)

    if rank == 0 and not multi and not args.no_extras:
        from oracle import vx_oracle as oracle
        try:
            line["decode_batch16"] = bench_decode_batch(torch, llama, shape, peaks, 16)
            line["decode_fp8"] = bench_decode_quant(torch, llama, shape, peaks, "fp8")
            line["decode_q4"] = bench_decode_quant(torch, llama, shape, peaks, "q4")
            line["moe_experts_q4"] = bench_moe_experts(torch)
            line["gemm_f32_1024"] = bench_gemm_f32(torch, oracle)
            line["small_llama_f32"] = bench_small_llama(torch, oracle, llama)
            # attention before the big GEMMs: seconds of dense GEMM leave the GPU
            # at its power cap, and what runs next is measured at lower clocks
            line["flash_attention"] = bench_flash(torch, oracle, peaks)
            line["gemm"] = bench_gemm(torch, oracle, peaks)
            # the other sizes of the GEMM configuration (2048 fits L2: noted)
            line["gemm_sweep"] = {}
            for n, it in ((2048, 50), (4096, 30), (16384, 5)):
                r = bench_gemm(torch, oracle, peaks, n=n, iters=it, check_rows=4)
                # a single product of the small sizes is mostly launch latency:
                # the better of the two timings
                line["gemm_sweep"][str(n)] = dict(
                    tflops=round(max(r["tflops"], r["tflops_back_to_back"]), 1),
                    rel_err_sampled_rows=r["rel_err_sampled_rows"],
                    kernel_status=r["kernel_status"])
        except RuntimeError as e:        # reported, never hidden
            line["extras_error"] = str(e)
    if rank == 0:
        if host_model is not None:
            from oracle import vx_oracle as oracle
            line["cpu_baseline"] = cpu_baseline_with_the_model(
                oracle, host_model, said, os.cpu_count() or 1)
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
                    help="skip the GEMM, flash-attention and batch-16 figures")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
