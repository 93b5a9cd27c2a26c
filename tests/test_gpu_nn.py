"""Every std::nn operator through its vx_nn_* export against the CPU oracle, on
the shapes, random data and criterion of the reference's own parity test
(tests/optimizations/pass/std_nn_kernels_match_loops_on_the_cpu.vx:101-115,
425-445): max |got - want| <= 1e-5 * max |want|."""
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


def rand_bf16(oracle, n, seed, scale):
    return oracle.f32_to_bf16(oracle.random_f32(n, seed, scale))


@pytest.mark.parametrize("rows,cols", [(300, 896), (64, 4864), (7, 8), (1, 1032)])
def test_matvec_and_add(oracle, rows, cols):
    w = rand_bf16(oracle, rows * cols, 11, 0.1)
    x = oracle.random_f32(cols, 12, 1.0)
    y0 = oracle.random_f32(rows, 13, 1.0)
    tw, tx = dev(w, True), dev(x)
    ty = abi.DeviceTensor.empty((rows,), abi.F32)
    ops.nn_matvec(ty, tw, tx, rows, cols)
    wf = oracle.bf16_to_f32(w).astype(np.float64).reshape(rows, cols)
    close(ty.to_host(), wf @ x.astype(np.float64))
    ta = dev(y0)
    ops.nn_matvec_add(ta, tw, tx, rows, cols)
    close(ta.to_host(), y0 + wf @ x.astype(np.float64))
    # and bit-for-bit order independence is not claimed: the f32 oracle agrees
    close(ty.to_host(), oracle.nn_matvec(w, x, rows, cols), 2e-6)


def test_matvec_heads_add(oracle):
    rows, heads, hd = 200, 14, 64
    cols = heads * hd
    w = rand_bf16(oracle, rows * cols, 31, 0.1)
    x = oracle.random_f32(cols, 32, 1.0).reshape(heads, hd)
    y0 = oracle.random_f32(rows, 33, 1.0)
    ty = dev(y0)
    ops.nn_matvec_heads_add(ty, dev(w, True), dev(x), rows, heads, hd)
    wf = oracle.bf16_to_f32(w).astype(np.float64).reshape(rows, cols)
    close(ty.to_host(), y0 + wf @ x.reshape(-1).astype(np.float64))


def test_qkv(oracle):
    qh, kvh, hd, cols = 14, 2, 64, 896
    rows = (qh + 2 * kvh) * hd
    w = rand_bf16(oracle, rows * cols, 21, 0.1)
    b = rand_bf16(oracle, rows, 22, 1.0)
    x = oracle.random_f32(cols, 23, 1.0)
    tq = abi.DeviceTensor.empty((qh, hd), abi.F32)
    tk = abi.DeviceTensor.empty((kvh, hd), abi.F32)
    tv = abi.DeviceTensor.empty((kvh, hd), abi.F32)
    ops.nn_qkv(tq, tk, tv, dev(w, True), dev(b, True), dev(x), qh, kvh, hd, cols)
    wf = oracle.bf16_to_f32(w).astype(np.float64).reshape(rows, cols)
    want = wf @ x.astype(np.float64) + oracle.bf16_to_f32(b)
    got = np.concatenate([t.to_host().reshape(-1) for t in (tq, tk, tv)])
    close(got, want)


def test_swiglu(oracle):
    rows, cols = 200, 896
    w = rand_bf16(oracle, 2 * rows * cols, 41, 0.1)
    x = oracle.random_f32(cols, 42, 1.0)
    tout = abi.DeviceTensor.empty((rows,), abi.F32)
    ops.nn_swiglu(tout, dev(w, True), dev(x), rows, cols)
    wf = oracle.bf16_to_f32(w).astype(np.float64).reshape(2 * rows, cols)
    g = wf[:rows] @ x.astype(np.float64)
    u = wf[rows:] @ x.astype(np.float64)
    close(tout.to_host(), g / (1.0 + np.exp(-g)) * u)


@pytest.mark.parametrize("n", [896, 3584, 8, 1025])
def test_rms_norm(oracle, n):
    x = oracle.random_f32(n, 45, 3.0)
    w = rand_bf16(oracle, n, 46, 1.0)
    ty = abi.DeviceTensor.empty((n,), abi.F32)
    ops.nn_rms_norm(ty, dev(x), dev(w, True), n, 1e-6)
    xd = x.astype(np.float64)
    want = xd / np.sqrt((xd * xd).mean() + 1e-6) * oracle.bf16_to_f32(w)
    close(ty.to_host(), want)


@pytest.mark.parametrize("qh,kvh,hd,pos,max_seq", [(14, 2, 64, 5, 16),
                                                   (28, 4, 128, 300, 400)])
def test_rope_and_store(oracle, qh, kvh, hd, pos, max_seq):
    cos, sin = oracle.rope_tables(max_seq, hd, 1000000.0)
    q = oracle.random_f32(qh * hd, 51, 1.0).reshape(qh, hd)
    k = oracle.random_f32(kvh * hd, 52, 1.0).reshape(kvh, hd)
    v = oracle.random_f32(kvh * hd, 53, 1.0).reshape(kvh, hd)
    kc = np.zeros((max_seq, kvh, hd), np.float32)
    vc = np.zeros((max_seq, kvh, hd), np.float32)
    want_q = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, pos)
    tq = abi.DeviceTensor.empty((qh, hd), abi.F32)
    tkc = dev(np.zeros_like(kc))
    tvc = dev(np.zeros_like(vc))
    ops.nn_rope_and_store(tq, tkc, tvc, dev(q), dev(k), dev(v), dev(cos),
                          dev(sin), pos, qh, kvh, hd)
    # two products and one sum per value, each rounded once: the same bits
    assert np.array_equal(tq.to_host(), want_q)
    assert np.array_equal(tkc.to_host(), kc)
    assert np.array_equal(tvc.to_host(), vc)


ATTENTION_CASES = [  # q_heads, kv_heads, head_dim, pos, max_seq
    (14, 2, 64, 37, 64), (28, 4, 128, 300, 400), (14, 2, 64, 0, 8),
    (32, 2, 64, 199, 256), (32, 4, 128, 1000, 1024), (28, 4, 128, 699, 768),
    (32, 2, 64, 655, 704), (32, 32, 128, 639, 640), (6, 6, 96, 31, 32)]


@pytest.fixture(params=[1, 2], ids=["cluster", "split"])
def attention_kernel(request):
    """Both attention kernels: the cluster merge (the default) and the
    reference's split scheme with partial results in `part` and a counter per
    head tile (nn.vx:343-368, 823-866)."""
    from vx_b200.lib import lib
    before = lib().vx_b200_attention_kernel(request.param)
    yield request.param
    lib().vx_b200_attention_kernel(before)


@pytest.mark.parametrize("qh,kvh,hd,pos,max_seq", ATTENTION_CASES)
def test_attention(oracle, attention_kernel, qh, kvh, hd, pos, max_seq):
    q = oracle.random_f32(qh * hd, 61, 2.0).reshape(qh, hd)
    kc = oracle.random_f32(max_seq * kvh * hd, 62, 2.0).reshape(max_seq, kvh, hd)
    vc = oracle.random_f32(max_seq * kvh * hd, 63, 1.0).reshape(max_seq, kvh, hd)
    shape = ops.nn_attention_scratch_shape(max_seq, qh, kvh, hd)
    part = dev(np.full(shape, np.nan, np.float32))   # scratch content is free
    out = abi.DeviceTensor.empty((qh, hd), abi.F32)
    tq, tk, tv = dev(q), dev(kc), dev(vc)
    # twice at this position and once at an earlier one in between: the split
    # kernel's counters must be back at zero after every launch, whatever the
    # number of parts was
    for p in (pos, pos // 3, pos):
        ops.nn_attention(out, part, tq, tk, tv, p, qh, kvh, hd)
        close(out.to_host(), oracle.attention_f64(q, kc, vc, p))
    close(out.to_host(), oracle.nn_attention(q, kc, vc, pos), 2e-5)


def test_attention_after_a_run_of_cache_writes(oracle, attention_kernel):
    """The cache filled by back-to-back nn_rope_and_store calls (short kernels
    that each let their successor start early) and attended at once: every row
    must be the written one."""
    qh, kvh, hd, max_seq = 8, 2, 64, 48
    cos, sin = oracle.rope_tables(max_seq, hd, 10000.0)
    kc = np.zeros((max_seq, kvh, hd), np.float32)
    vc = np.zeros_like(kc)
    tkc, tvc = dev(np.full_like(kc, np.nan)), dev(np.full_like(vc, np.nan))
    tcos, tsin = dev(cos), dev(sin)
    tq = abi.DeviceTensor.empty((qh, hd), abi.F32)
    part = abi.DeviceTensor.empty(
        ops.nn_attention_scratch_shape(max_seq, qh, kvh, hd), abi.F32)
    out = abi.DeviceTensor.empty((qh, hd), abi.F32)
    steps = []
    for pos in range(40):
        q = oracle.random_f32(qh * hd, 500 + pos, 1.0).reshape(qh, hd)
        k = oracle.random_f32(kvh * hd, 600 + pos, 1.0).reshape(kvh, hd)
        v = oracle.random_f32(kvh * hd, 700 + pos, 1.0).reshape(kvh, hd)
        steps.append((dev(q), dev(k), dev(v)))
        want_q = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, pos)
    for pos, (dq, dk, dv) in enumerate(steps):
        ops.nn_rope_and_store(tq, tkc, tvc, dq, dk, dv, tcos, tsin, pos, qh, kvh, hd)
    ops.nn_attention(out, part, tq, tkc, tvc, 39, qh, kvh, hd)
    close(out.to_host(), oracle.attention_f64(want_q, kc, vc, 39))


def test_argmax_known_answer(oracle):
    # "nn_argmax of 151936: 50645": two equal largest values, the lower index.
    n = 151936
    h = oracle.random_f32(n, 71, 1.0)
    h[n - 7] = 3.0
    h[n // 3] = 3.0
    out = abi.DeviceTensor.empty((1,), abi.I32)
    ops.nn_argmax(out, dev(h), n)
    assert int(out.to_host()[0]) == 50645 == oracle.nn_argmax(h)


def test_embed(oracle):
    rows, dim, token = 10, 896, 7
    table = rand_bf16(oracle, rows * dim, 81, 1.0)
    x = abi.DeviceTensor.empty((dim,), abi.F32)
    ops.nn_embed(x, dev(table, True), dev(np.array([token], np.int32)), dim)
    assert np.array_equal(x.to_host(), oracle.nn_embed(table, token, dim))


# ---- kernels for n positions at once: every row bit for bit the one-position
# ---- kernel's (the method and sizes of the reference's
# ---- apple_gpu_kernels_for_n_positions_match_one_position.vx: 5 positions)
def test_rows_kernels_match_one_position_bit_for_bit(oracle):
    n = 5
    # bf16 product: 16 rows of 1024
    rows, cols = 16, 1024
    w = rand_bf16(oracle, rows * cols, 91, 0.1)
    x = oracle.random_f32(n * cols, 92, 1.0).reshape(n, cols)
    tw = dev(w, True)
    ty = abi.DeviceTensor.empty((n, rows), abi.F32)
    ops.nn_matvec_rows(ty, tw, dev(x), n, rows, cols)
    got = ty.to_host()
    for t in range(n):
        one = abi.DeviceTensor.empty((rows,), abi.F32)
        ops.nn_matvec(one, tw, dev(x[t]), rows, cols)
        assert np.array_equal(got[t], one.to_host()), t
    # Q4_0 product: 64 rows of 512
    rows, cols = 64, 512
    wq, sq = oracle.quant_inputs("q4", rows, cols, 93)
    xq = oracle.random_f32(n * cols, 94, 1.0).reshape(n, cols)
    twq, tsq = dev(wq), dev(sq)
    tyq = abi.DeviceTensor.empty((n, rows), abi.F32)
    ops.nn_matvec_q4_rows(tyq, twq, tsq, dev(xq), n, rows, cols)
    gotq = tyq.to_host()
    for t in range(n):
        one = abi.DeviceTensor.empty((rows,), abi.F32)
        ops.nn_matvec_quant("q4", one, twq, tsq, dev(xq[t]), rows, cols)
        assert np.array_equal(gotq[t], one.to_host()), t
    # rms norm: 256 values a row
    dim = 256
    xn = oracle.random_f32(n * dim, 95, 3.0).reshape(n, dim)
    wn = rand_bf16(oracle, dim, 96, 1.0)
    tn = abi.DeviceTensor.empty((n, dim), abi.F32)
    ops.nn_rms_norm_rows(tn, dev(xn), dev(wn, True), n, dim, 1e-6)
    gotn = tn.to_host()
    for t in range(n):
        one = abi.DeviceTensor.empty((dim,), abi.F32)
        ops.nn_rms_norm(one, dev(xn[t]), dev(wn, True), dim, 1e-6)
        assert np.array_equal(gotn[t], one.to_host()), t
    # embed and argmax
    table = rand_bf16(oracle, 10 * dim, 97, 1.0)
    tokens = np.array([7, 0, 9, 3, 3], np.int32)
    te = abi.DeviceTensor.empty((n, dim), abi.F32)
    ops.nn_embed_rows(te, dev(table, True), dev(tokens), n, dim)
    assert np.array_equal(te.to_host(), oracle.bf16_to_f32(table).reshape(10, dim)[tokens])
    logits = oracle.random_f32(n * 3000, 98, 1.0).reshape(n, 3000)
    logits[2, 17] = logits[2, 2900] = 5.0                # a tie: the lower index
    ta = abi.DeviceTensor.empty((n,), abi.I32)
    ops.nn_argmax_rows(ta, dev(logits), n, 3000)
    assert list(ta.to_host()) == [int(np.argmax(r)) for r in logits]
