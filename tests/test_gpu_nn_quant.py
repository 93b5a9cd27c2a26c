"""The fp8 and Q4_0 projections through their vx_nn_* exports, on the shapes,
codes, scales and criterion of the reference's own tests
(tests/optimizations/pass/std_nn_fp8_kernels_match_loops_on_the_cpu.vx and
std_nn_q4_kernels_match_loops_on_the_cpu.vx): max |got - want| <= 1e-5 * max
|want| against plain f64 loops over the definition of each format."""
import numpy as np
import pytest

from vx_b200 import abi, ops

pytestmark = pytest.mark.gpu


def close(got, want, tol=1e-5):
    want = np.asarray(want, np.float64)
    worst = np.abs(np.asarray(got, np.float64) - want).max()
    assert worst <= tol * np.abs(want).max(), (worst, np.abs(want).max())


def dev(a, bf16=False):
    return abi.DeviceTensor.from_host(a, bf16=bf16)


@pytest.mark.parametrize("quant", ["fp8", "q4"])
@pytest.mark.parametrize("rows,cols", [(296, 896), (64, 4864), (8, 128),
                                       (4096, 4096),
                                       # a last tile of six row pairs; more
                                       # 16-row tiles than the GPU has warps
                                       (300, 512), (40960, 256)])
def test_matvec_and_add(oracle, quant, rows, cols):
    w, s = oracle.quant_inputs(quant, rows, cols, 1)
    x = oracle.random_f32(cols, 3, 1.0)
    y0 = oracle.random_f32(rows, 4, 1.0)
    want = oracle.quant_dot_f64(quant, w, s, x, rows, cols)
    tw, ts, tx = dev(w), dev(s), dev(x)
    ty = abi.DeviceTensor.empty((rows,), abi.F32)
    ops.nn_matvec_quant(quant, ty, tw, ts, tx, rows, cols)
    close(ty.to_host(), want)
    # the restatement of the reference kernel agrees to rounding
    close(ty.to_host(), oracle.quant_matvec(quant, w, s, x, rows, cols), 4e-6)
    ta = dev(y0)
    ops.nn_matvec_quant(quant, ta, tw, ts, tx, rows, cols, add=True)
    close(ta.to_host(), y0 + want)


@pytest.mark.parametrize("quant,rows,heads,hd", [("fp8", 200, 14, 64),
                                                 ("q4", 200, 32, 128),
                                                 ("q4", 64, 28, 40)])
def test_matvec_heads_add(oracle, quant, rows, heads, hd):
    cols = heads * hd
    w, s = oracle.quant_inputs(quant, rows, cols, 11)
    x = oracle.random_f32(cols, 13, 1.0)
    y0 = oracle.random_f32(rows, 14, 1.0)
    ty = dev(y0)
    ops.nn_matvec_quant_heads_add(quant, ty, dev(w), dev(s), dev(x.reshape(heads, hd)),
                                  rows, heads, hd)
    close(ty.to_host(), y0 + oracle.quant_dot_f64(quant, w, s, x, rows, cols))


@pytest.mark.parametrize("quant,cols", [("fp8", 896), ("q4", 2560)])
def test_qkv(oracle, quant, cols):
    qh, kvh, hd = 14, 2, 64
    rows = (qh + 2 * kvh) * hd
    w, s = oracle.quant_inputs(quant, rows, cols, 21)
    x = oracle.random_f32(cols, 23, 1.0)
    b = oracle.f32_to_bf16(oracle.random_f32(rows, 24, 4.0))
    tq = abi.DeviceTensor.empty((qh, hd), abi.F32)
    tk = abi.DeviceTensor.empty((kvh, hd), abi.F32)
    tv = abi.DeviceTensor.empty((kvh, hd), abi.F32)
    ops.nn_qkv_quant(quant, tq, tk, tv, dev(w), dev(s), dev(b, True), dev(x), qh,
                     kvh, hd, cols)
    want = oracle.quant_dot_f64(quant, w, s, x, rows, cols) + oracle.bf16_to_f32(b)
    got = np.concatenate([t.to_host().reshape(-1) for t in (tq, tk, tv)])
    nq, nkv = qh * hd, kvh * hd
    for lo, hi in ((0, nq), (nq, nq + nkv), (nq + nkv, rows)):   # q, k, v apart
        close(got[lo:hi], want[lo:hi])


@pytest.mark.parametrize("quant,rows,cols", [("fp8", 200, 896), ("q4", 200, 4864)])
def test_swiglu(oracle, quant, rows, cols):
    w, s = oracle.quant_inputs(quant, 2 * rows, cols, 31)
    x = oracle.random_f32(cols, 33, 1.0)
    tout = abi.DeviceTensor.empty((rows,), abi.F32)
    ops.nn_swiglu_quant(quant, tout, dev(w), dev(s), dev(x), rows, cols)
    both = oracle.quant_dot_f64(quant, w, s, x, 2 * rows, cols)
    g, u = both[:rows], both[rows:]
    close(tout.to_host(), g / (1.0 + np.exp(-g)) * u)
    close(tout.to_host(), oracle.quant_swiglu(quant, w, s, x, rows, cols), 4e-6)


def test_every_fp8_code(oracle):
    """Each non-NaN code alone in a row with scale 1 and x = 1: the hardware
    conversion must give the value of the f8e4m3 definition, bit for bit."""
    codes = [c for c in range(256) if (c & 127) != 127]
    rows, cols = len(codes) + (-len(codes)) % 4, 128
    w = np.zeros(rows * cols // 4, np.uint32)
    for r, c in enumerate(codes):
        w[r * cols // 4] = c
    s = np.ones(((rows + 127) // 128) * (cols // 128), np.float32)
    x = np.zeros(cols, np.float32)
    x[0] = 1.0
    ty = abi.DeviceTensor.empty((rows,), abi.F32)
    ops.nn_matvec_quant("fp8", ty, dev(w), dev(s), dev(x), rows, cols)
    want = oracle.quant_dot_f64("fp8", w, s, x, rows, cols)
    assert np.array_equal(ty.to_host().astype(np.float64), want)


# ---- a mixture-of-experts layer (nn.vx:899-1066, 2104-2262) ---------------------------
def test_top_k(oracle):
    for n, k, seed in ((128, 8, 5), (256, 4, 6), (60, 60, 7), (1, 1, 8)):
        logits = oracle.random_f32(n, seed, 3.0)
        if n > 100:
            logits[90] = logits[11] = 9.0         # equal largest: index 11 first
        tid = abi.DeviceTensor.empty((k,), abi.I32)
        tw = abi.DeviceTensor.empty((k,), abi.F32)
        ops.nn_top_k(tid, tw, dev(logits), n, k)
        ids, weights = oracle.nn_top_k(logits, k)
        assert np.array_equal(tid.to_host(), ids), (n, k)
        close(tw.to_host(), weights, 2e-6)


@pytest.mark.parametrize("quant,experts,k,inter,hidden", [
    ("q4", 32, 8, 96, 512), ("q4", 8, 4, 1056, 2080), ("bf16", 16, 4, 200, 896)])
def test_moe_swiglu_and_down(oracle, quant, experts, k, inter, hidden):
    """The two expert projections of one token on the reference's own cases
    (std_nn_q4_kernels_match_loops_on_the_cpu.vx: 8 of 32 experts 96 x 512, 4
    of 8 experts 1056 x 2080) and a bf16 one, against f64 loops; the down
    projection takes the GPU's own activations, as the reference's test does."""
    ids = np.array([((experts - 1 - e * 5) % experts + experts) % experts
                    for e in range(k)], np.int32)
    weights = (np.float32(0.5) + oracle.random_f32(k, 75, 0.4)).astype(np.float32)
    x = oracle.random_f32(hidden, 76, 1.0)
    y0 = oracle.random_f32(hidden, 77, 1.0)
    if quant == "q4":
        gu, gu_s = oracle.quant_inputs("q4", experts * 2 * inter, hidden, 71)
        dn, dn_s = oracle.quant_inputs("q4", experts * hidden, inter, 73)
        gu_rows = oracle.quant_dot_f64("q4", gu, gu_s, x, experts * 2 * inter, hidden)
        t_gu, t_gus, t_dn, t_dns = dev(gu), dev(gu_s), dev(dn), dev(dn_s)
    else:
        gu = oracle.f32_to_bf16(oracle.random_f32(experts * 2 * inter * hidden, 71, 0.1))
        dn = oracle.f32_to_bf16(oracle.random_f32(experts * hidden * inter, 73, 0.1))
        gu_rows = oracle.bf16_to_f32(gu).astype(np.float64) \
            .reshape(experts * 2 * inter, hidden) @ x.astype(np.float64)
        t_gu, t_gus, t_dn, t_dns = dev(gu, True), None, dev(dn, True), None
    act = abi.DeviceTensor.empty((k, inter), abi.F32)
    ops.nn_moe_swiglu(act, t_gu, dev(ids), dev(x), k, inter, hidden, experts,
                      scales=t_gus)
    got_a = act.to_host()
    want_a = np.empty((k, inter))
    for e in range(k):
        g = gu_rows[ids[e] * 2 * inter:ids[e] * 2 * inter + inter]
        u = gu_rows[ids[e] * 2 * inter + inter:(ids[e] + 1) * 2 * inter]
        want_a[e] = g / (1.0 + np.exp(-g)) * u
    close(got_a.reshape(-1), want_a.reshape(-1))
    ty = dev(y0)
    ops.nn_moe_down_add(ty, t_dn, dev(ids), dev(weights), act, k, hidden, inter,
                        experts, scales=t_dns)
    want_y = y0.astype(np.float64)
    for e in range(k):
        if quant == "q4":
            rows = oracle.quant_dot_f64("q4", dn, dn_s, got_a[e], experts * hidden,
                                        inter)[ids[e] * hidden:(ids[e] + 1) * hidden]
        else:
            rows = oracle.bf16_to_f32(dn).astype(np.float64) \
                .reshape(experts * hidden, inter)[ids[e] * hidden:(ids[e] + 1) * hidden] \
                @ got_a[e].astype(np.float64)
        want_y = want_y + float(weights[e]) * rows
    close(ty.to_host(), want_y)
    assert ops.kernel_status() == 0
