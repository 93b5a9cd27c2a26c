"""The CPU oracle against every known answer the reference's own tests hold for
this path (no GPU)."""
import numpy as np
import pytest


def test_gpu_matmul_roles_known_answer(oracle):
    # tests/backend/pass/gpu_matmul_roles.vx EXPECT: 38 56 83 128 9 7 10
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    b = np.arange(1, 13, dtype=np.float32).reshape(3, 4)
    c = oracle.gemm(a, b)
    assert [c[0, 0], c[0, 3], c[1, 0], c[1, 3]] == [38, 56, 83, 128]
    p = np.arange(1, 10, dtype=np.float32).reshape(3, 3)
    q = np.diag(np.arange(1, 4, dtype=np.float32))
    r = oracle.gemm(p, q)
    assert [r[0, 2], r[2, 0], r[1, 1]] == [9, 7, 10]
    # the wrong assignments that the test is built to expose give other numbers
    wrong = oracle.gemm(q, p)
    assert [wrong[0, 2], wrong[2, 0], wrong[1, 1]] == [3, 21, 10]


def test_gpu_matmul_dtypes_known_answer(oracle):
    # tests/backend/pass/gpu_matmul_dtypes.vx EXPECT: 19 50 197 4032
    a = np.array([[1, 2], [3, 4]], dtype=np.float64)
    b = np.array([[5, 6], [7, 8]], dtype=np.float64)
    c = oracle.gemm(a, b)
    assert (c[0, 0], c[1, 1]) == (19, 50)
    e = np.eye(64, dtype=np.float32)
    m = np.arange(64 * 64, dtype=np.float32).reshape(64, 64)
    r = oracle.gemm(e, m)
    assert (r[3, 5], r[63, 0]) == (197, 4032)


def test_matmul_into_buffer_and_execution(oracle):
    # matmul_into_buffer.vx EXPECT: 3 7 3 7; benchmarks/matmul_execution.vx: 24
    w = np.array([[1, 2], [3, 4]], dtype=np.float32)
    y = oracle.gemm(w, np.ones((2, 1), np.float32))
    assert [y[0, 0], y[1, 0]] == [3, 7]
    c = oracle.gemm(np.full((4, 4), 2, np.float32), np.full((4, 4), 3, np.float32))
    assert (c == 24).all()


def test_the_two_gemm_loops_give_the_same_bits(oracle):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (96, 200)).astype(np.float32)
    b = rng.uniform(-1, 1, (200, 72)).astype(np.float32)
    assert np.array_equal(oracle.gemm(a, b), oracle.gemm(a, b, fast=True))


def test_flat_matvec_is_the_gemm_with_one_column(oracle):
    rng = np.random.default_rng(1)
    w = rng.uniform(-1, 1, (50, 64)).astype(np.float32)
    x = rng.uniform(-1, 1, 64).astype(np.float32)
    assert np.array_equal(oracle.matvec_f32(w, x),
                          oracle.gemm(w, x.reshape(-1, 1)).reshape(-1))


def test_bf16_rounding_is_nearest_even(oracle):
    # exact RNE, NaN stays NaN, the largest finite value rounds to infinity
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.4028235e38,
                  np.inf, 3.3895314e38], dtype=np.float32)
    got = oracle.f32_to_bf16(x)
    assert list(got[:4]) == [0x3F80, 0x3F80, 0x3F82, 0xBF80]
    assert got[4] == 0x7F80 and got[5] == 0x7F80
    assert got[6] == 0x7F7F                      # the largest finite bf16
    nan = oracle.f32_to_bf16(np.array([np.nan], np.float32))
    assert np.isnan(oracle.bf16_to_f32(nan)[0])
    # round trip of every bf16 pattern that is not a NaN
    every = np.arange(65536, dtype=np.uint16)
    f = oracle.bf16_to_f32(every)
    keep = ~np.isnan(f)
    assert np.array_equal(oracle.f32_to_bf16(f)[keep], every[keep])


def test_small_integer_gemm_is_exact(oracle):
    # benchmarks/gpu_gemm/cublas_gemm.cu:22-28: sums of small integers are exact
    m, n, k = 64, 48, 512
    a = ((np.arange(m)[:, None] * 3 + np.arange(k)[None, :] * 5) % 7 - 3).astype(np.float32)
    b = ((np.arange(k)[:, None] * 2 + np.arange(n)[None, :]) % 5 - 2).astype(np.float32)
    a16, b16 = oracle.f32_to_bf16(a), oracle.f32_to_bf16(b)
    exact = a.astype(np.int64) @ b.astype(np.int64)
    assert oracle.gemm_bf16_entry(a16, b16, 5, 7) == exact[5, 7]
    rows = np.arange(m, dtype=np.int64)
    got = oracle.bf16_to_f32(oracle.gemm_bf16_rows(a16, b16, rows))
    want = oracle.bf16_to_f32(oracle.f32_to_bf16(exact.astype(np.float32)))
    assert np.array_equal(got, want)


def test_nn_argmax_known_answer(oracle):
    # std_nn_kernels_match_loops_on_the_cpu.vx:39 "nn_argmax of 151936: 50645"
    n = 151936
    h = oracle.random_f32(n, 71, 1.0)
    assert -1.0 <= h.min() and h.max() < 1.0
    h[n - 7] = 3.0
    h[n // 3] = 3.0
    assert oracle.nn_argmax(h) == 50645


def test_random_matches_its_definition(oracle):
    # mix / random of the same file, :45-60, restated in Python integers
    def mix(x):
        h = (x * 2654435761) & 0xFFFFFFFF
        h ^= h >> 15
        h = (h * 2246822519) & 0xFFFFFFFF
        h ^= h >> 13
        return h
    got = oracle.random_f32(100, 61, 2.0)
    for i in (0, 1, 17, 99):
        u = np.float32(mix((61 * 7919 + i) & 0xFFFFFFFF) >> 8)
        want = (u * np.float32(0.00000011920929) - np.float32(1.0)) * np.float32(2.0)
        assert got[i] == want


def test_nn_ops_meet_the_reference_criterion(oracle):
    """The f32 kernels-order oracle against f64 loops, with the reference test's
    shapes and its bound 1e-5 * max|want| (:101-115)."""
    def close(got, want):
        want = np.asarray(want, np.float64)
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()

    rows, cols = 300, 896
    w = oracle.f32_to_bf16(oracle.random_f32(rows * cols, 11, 0.1))
    x = oracle.random_f32(cols, 12, 1.0)
    wf = oracle.bf16_to_f32(w).astype(np.float64).reshape(rows, cols)
    close(oracle.nn_matvec(w, x, rows, cols), wf @ x.astype(np.float64))
    g = wf[:150] @ x.astype(np.float64)
    u = wf[150:] @ x.astype(np.float64)
    close(oracle.nn_swiglu(w, x, 150, cols), g / (1 + np.exp(-g)) * u)
    xn = oracle.random_f32(3584, 45, 3.0)
    wn = oracle.f32_to_bf16(oracle.random_f32(3584, 46, 1.0))
    xd = xn.astype(np.float64)
    close(oracle.nn_rms_norm(xn, wn, 3584, 1e-6),
          xd / np.sqrt((xd * xd).mean() + 1e-6) * oracle.bf16_to_f32(wn))
    for qh, kvh, hd, pos, max_seq in [(14, 2, 64, 37, 64), (32, 2, 64, 655, 704),
                                      (28, 4, 128, 699, 768), (14, 2, 64, 0, 8)]:
        q = oracle.random_f32(qh * hd, 61, 2.0).reshape(qh, hd)
        kc = oracle.random_f32(max_seq * kvh * hd, 62, 2.0).reshape(max_seq, kvh, hd)
        vc = oracle.random_f32(max_seq * kvh * hd, 63, 1.0).reshape(max_seq, kvh, hd)
        close(oracle.nn_attention(q, kc, vc, pos),
              oracle.attention_f64(q, kc, vc, pos))


def test_rope_is_a_rotation(oracle):
    qh, kvh, hd, pos, max_seq = 4, 2, 64, 5, 16
    cos, sin = oracle.rope_tables(max_seq, hd, 10000.0)
    q = oracle.random_f32(qh * hd, 51, 1.0).reshape(qh, hd)
    k = oracle.random_f32(kvh * hd, 52, 1.0).reshape(kvh, hd)
    v = oracle.random_f32(kvh * hd, 53, 1.0).reshape(kvh, hd)
    kc = np.zeros((max_seq, kvh, hd), np.float32)
    vc = np.zeros_like(kc)
    qr = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, pos)
    assert np.allclose(np.linalg.norm(qr, axis=1), np.linalg.norm(q, axis=1), rtol=1e-6)
    assert np.array_equal(vc[pos], v) and not kc[pos + 1].any()
    # position 0 turns nothing
    q0 = oracle.nn_rope_and_store(kc, vc, q, k, v, cos, sin, 0)
    assert np.array_equal(q0, q)


def test_llama_generate_is_deterministic_and_causal(oracle):
    cfg = oracle.LlamaConfig(64, 176, 2, 4, 4, 512, 32)
    n = oracle.llama_weight_count(cfg)
    w = (np.random.default_rng(42).standard_normal(n, dtype=np.float32) * 0.02).astype(np.float32)
    a = oracle.llama_generate(cfg, w, 1, 12)
    b = oracle.llama_generate(cfg, w, 1, 20)
    assert a[0] == 1 and np.array_equal(a, b[:13])
    assert ((0 <= b) & (b < 512)).all()


def test_attention_rows_causal_prefix_property(oracle):
    """Row i of causal attention over S rows equals row i over the first i+1."""
    rng = np.random.default_rng(10)
    S, D = 96, 32
    q, k, v = (oracle.f32_to_bf16(rng.standard_normal((S, D), dtype=np.float32))
               for _ in range(3))
    full = oracle.attention_rows(q, k, v, 0.17, True, np.array([40]))
    cut = oracle.attention_rows(q[:41], k[:41], v[:41], 0.17, False, np.array([40]))
    assert np.array_equal(full, cut)


def test_all_reduce_adds_in_rank_order(oracle):
    parts = [np.full(5, 0.1 * (r + 1), np.float32) for r in range(4)]
    want = ((parts[0] + parts[1]) + parts[2]) + parts[3]
    assert np.array_equal(oracle.all_reduce_sum_f32(parts), want)


def test_the_two_restatements_of_the_llama_decode_give_the_same_100_tokens(oracle):
    """Config 2 (dim 288, 6 layers, 6 heads, hidden 768, vocab 32000, seq 256,
    N(0, 0.02^2) from seed 42, greedy from BOS = 1): the restatement of
    tests/backend/pass/llama2.vx (two-pass softmax, vx_oracle.cpp) and the
    independent one of benchmarks/llama2_100.vx (online softmax,
    llama_twin.c) are two programs the reference expects the same text from.
    They share no code here and must give the same 100 tokens."""
    from vx_b200 import llama
    flat, _ = llama.small_f32_weights()
    cfg = oracle.LlamaConfig(288, 768, 6, 6, 6, 32000, 256)
    first, gaps = oracle.llama_generate(cfg, flat, 1, 100, want_gaps=True)
    second = oracle.llama_twin_generate(cfg, flat, 1, 100)
    differ = [i for i in range(101) if first[i] != second[i]]
    assert not differ, "first difference at step %d (top-2 logit gap %.3g)" % (
        differ[0] - 1, gaps[differ[0] - 1])
    # a random model with a shared embedding/classifier mostly repeats itself;
    # the sequence still changes token several times
    assert len(set(first.tolist())) >= 3


@pytest.mark.parametrize("quant,rows,cols", [("fp8", 296, 896), ("fp8", 64, 4864),
                                             ("q4", 296, 896), ("q4", 64, 4864)])
def test_quantised_matvec_meets_the_reference_criterion(oracle, quant, rows, cols):
    """The restatements of nn_matvec_fp8 / nn_matvec_q4 on the shapes, codes and
    scales of the reference's tests
    (std_nn_{fp8,q4}_kernels_match_loops_on_the_cpu.vx), against the plain f64
    loops of those tests, with their criterion."""
    w, s = oracle.quant_inputs(quant, rows, cols, 1)
    x = oracle.random_f32(cols, 3, 1.0)
    want = oracle.quant_dot_f64(quant, w, s, x, rows, cols)
    got = oracle.quant_matvec(quant, w, s, x, rows, cols)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    y0 = oracle.random_f32(rows, 4, 1.0)
    got = oracle.quant_matvec(quant, w, s, x, rows, cols, y=y0)
    assert np.abs(got - (y0 + want)).max() <= 1e-5 * np.abs(y0 + want).max()


def test_fp8_code_values_follow_the_definition(oracle):
    """Each of the 254 non-NaN codes alone in a row: the table the kernels use
    (nn.vx:1316-1326) gives the value of the f8e4m3 definition exactly."""
    codes = [c for c in range(256) if (c & 127) != 127]
    rows, cols = len(codes) + (-len(codes)) % 4, 128
    w = np.zeros(rows * cols // 4, np.uint32)
    for r, c in enumerate(codes):
        w[r * cols // 4] = c                      # column 0 of row r
    s = np.ones(((rows + 127) // 128) * (cols // 128), np.float32)
    x = np.zeros(cols, np.float32)
    x[0] = 1.0
    got = oracle.quant_matvec("fp8", w, s, x, rows, cols)
    want = oracle.quant_dot_f64("fp8", w, s, x, rows, cols)
    assert np.array_equal(got.astype(np.float64), want)
    assert want[codes.index(0x38)] == 1.0 and want[codes.index(0x01)] == 2.0 ** -9
    assert want[codes.index(0x7e)] == 448.0 and want[codes.index(0xc0)] == -2.0


def test_top_k_orders_by_value_then_index(oracle):
    """nn_top_k (nn.vx:899-903): the k largest, the largest first, the lower
    index first of two equal values; weights = the softmax over those k."""
    logits = oracle.random_f32(200, 5, 3.0)
    logits[150] = logits[20] = 7.5            # equal largest: index 20 first
    logits[7] = -0.0
    logits[8] = 0.0
    ids, weights = oracle.nn_top_k(logits, 8)
    order = sorted(range(200), key=lambda i: (-float(logits[i]), i))[:8]
    assert list(ids) == order and list(ids[:2]) == [20, 150]
    e = np.exp(logits[ids].astype(np.float64) - float(logits[ids[0]]))
    assert np.abs(weights - e / e.sum()).max() <= 1e-6
    assert abs(float(weights.sum()) - 1.0) <= 1e-6


def test_moe_group_on_the_reference_cases(oracle):
    """The six cases of std_nn_moe_group_sorts_pairs_by_expert.vx. The plain
    stable sort (what that test calls `want`) and the restatement of the three
    kernels must agree, and the order must pass the test's `positions` check:
    every position names a distinct element."""
    for name, ids, experts, align in oracle.moe_group_reference_cases():
        want = oracle.moe_group(ids, experts, align)
        twin = oracle.moe_group_as_the_kernels(ids, experts, align)
        for key in want:
            assert np.array_equal(want[key], twin[key]), (name, key)
        n, order = ids.size, want["order"]
        room = n + experts * (align - 1)
        assert order.size == room, name
        at = np.full(n + room, -1)
        at[order] = np.arange(room)
        assert np.array_equal(at[order], np.arange(room)), name
        # each group: its pairs in rising order, all of its expert, then padding
        for e in range(experts):
            lo, hi = want["starts"][e], want["starts"][e + 1]
            assert lo % align == 0 and hi % align == 0, name
            members = order[lo:hi][order[lo:hi] < n]
            assert np.all(ids[members] == e) and np.all(np.diff(members) > 0), name
            assert members.size == np.count_nonzero(ids == e), name
            assert np.all(want["tile_expert"][lo // align:hi // align] == e), name
        assert np.all(want["tile_expert"][want["starts"][experts] // align:] == -1)
    # the sizes the cases are named for
    sizes = [(c[1].size, c[2], c[3]) for c in oracle.moe_group_reference_cases()]
    assert sizes == [(600, 5, 1), (1000, 160, 1), (1000, 160, 16), (300, 1, 1),
                     (2600, 40, 1), (2600, 40, 2)]


def test_moe_group_edges(oracle):
    for ids, experts, align in ((np.zeros(0, np.int32), 3, 4),
                                (np.array([2, 2, 2], np.int32), 3, 4),
                                (np.arange(256, dtype=np.int32) % 7, 7, 8),
                                (np.arange(257, dtype=np.int32) % 1024, 1024, 1)):
        want = oracle.moe_group(ids, experts, align)
        twin = oracle.moe_group_as_the_kernels(ids, experts, align)
        for key in want:
            assert np.array_equal(want[key], twin[key]), (ids.size, experts, key)
