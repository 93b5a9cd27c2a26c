"""The arithmetic facts the tensor-core routes for f32 data rest on, checked on
the CPU with numpy: an f32 value is the exact sum of three bf16 terms (the f32
GEMM, the prefill GEMMs, the batched and the Q4_0 projections), or of three f16
terms with the second and third scaled by 2^11 and 2^22 (the fp8 projections),
and the six largest of the nine term products are the product to f32 accuracy;
a Q4_0 code, a Q4_0 weight and an e4m3 code as exact bf16 values (the products
of many rows with quantised weights)."""
import numpy as np


def to_bf16(x):
    """Round f32 to bf16 (nearest even), returned as f32."""
    bits = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    return (rounded << 16).astype(np.uint32).view(np.float32)


def three_bf16(x):
    x = np.asarray(x, np.float32)
    t1 = to_bf16(x)
    r1 = (x - t1).astype(np.float32)
    t2 = to_bf16(r1)
    t3 = to_bf16((r1 - t2).astype(np.float32))
    return t1, t2, t3


def samples(seed, n=200000):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n) * np.exp(rng.uniform(-20, 20, n))
    return np.concatenate([x, [0.0, 1.0, -1.0, 3.0e38, 1.0e-30, 2.0 ** -126]]) \
        .astype(np.float32)


def test_three_bf16_terms_sum_to_the_value_exactly():
    x = samples(1)
    t1, t2, t3 = three_bf16(x)
    total = (t1.astype(np.float64) + t2.astype(np.float64)) + t3.astype(np.float64)
    assert np.array_equal(total.astype(np.float32), x)
    assert np.array_equal(total, x.astype(np.float64))        # nothing left over


def test_six_term_products_are_the_product_to_f32_accuracy():
    a, b = samples(2, 50000)[:50000], samples(3, 50000)[:50000]
    a, b = np.clip(a, -1e15, 1e15), np.clip(b, -1e15, 1e15)
    a1, a2, a3 = (t.astype(np.float64) for t in three_bf16(a))
    b1, b2, b3 = (t.astype(np.float64) for t in three_bf16(b))
    six = a1 * b1 + a1 * b2 + a2 * b1 + a1 * b3 + a2 * b2 + a3 * b1
    exact = a.astype(np.float64) * b.astype(np.float64)
    bound = 3.0 * 2.0 ** -24 * np.abs(exact) + 1e-300
    assert np.all(np.abs(six - exact) <= bound)


def test_three_scaled_f16_terms_sum_to_the_value_exactly():
    """h1 = f16(x), h2 = f16((x - h1) 2^11), h3 = f16(((x - h1) 2^11 - h2) 2^11):
    x = h1 + h2 2^-11 + h3 2^-22 for every f32 inside f16's range that is not
    tiny (activations after an RMSNorm are neither)."""
    rng = np.random.default_rng(4)
    x = (rng.standard_normal(200000) * np.exp(rng.uniform(-6, 9, 200000))) \
        .astype(np.float32)
    x = x[(np.abs(x) < 60000) & (np.abs(x) > 2.0 ** -10)]
    h1 = x.astype(np.float16)
    r1 = ((x - h1.astype(np.float32)) * np.float32(2048)).astype(np.float32)
    h2 = r1.astype(np.float16)
    r2 = ((r1 - h2.astype(np.float32)) * np.float32(2048)).astype(np.float32)
    h3 = r2.astype(np.float16)
    total = h1.astype(np.float64) + h2.astype(np.float64) / 2048 + \
        h3.astype(np.float64) / 4194304
    assert np.array_equal(total, x.astype(np.float64))


def test_a_q4_code_is_an_exact_bf16_after_the_magic_or():
    """0x4300 | code is the bf16 128 + code; less 136 it is code - 8."""
    codes = np.arange(16, dtype=np.uint32)
    as_f32 = ((0x4300 | codes) << 16).astype(np.uint32).view(np.float32)
    assert np.array_equal(as_f32, (128 + codes).astype(np.float32))
    assert np.array_equal(to_bf16(as_f32 - np.float32(136)),
                          (codes.astype(np.float32) - 8))


def bf16_bits_to_f64(bits):
    """The value of bf16 bit patterns (subnormals included), as f64."""
    bits = np.asarray(bits, np.uint32)
    return (bits << 16).astype(np.uint32).view(np.float32).astype(np.float64)


def test_a_q4_code_is_exact_in_bf16_through_the_bias_trick():
    """0x4300 | code is the bf16 128 + code (one unit in the last place at 128
    is 1), so subtracting 136 leaves code - 8: what the Q4_0 tensor-core kernels
    build their A operand from."""
    for code in range(16):
        biased = bf16_bits_to_f64(0x4300 | code)
        assert biased == 128.0 + code
        assert to_bf16(np.float32(biased - 136.0)) == np.float32(code - 8)
    assert bf16_bits_to_f64(0x4308) == 136.0


def test_a_q4_weight_is_the_exact_sum_of_two_bf16_terms():
    """(code - 8) * scale with an f16 scale has 4 + 11 significant bits: the
    first bf16 term and the rounded remainder hold all of them, for every code
    and every finite f16 scale. The prompt pass of a Q4_0 decoder rests on it."""
    scales = np.arange(0x0001, 0x7C00, dtype=np.uint16).view(np.float16) \
        .astype(np.float32)                                # every positive finite f16
    for code in range(16):
        v = (np.float32(code - 8) * scales).astype(np.float32)
        assert np.array_equal(v.astype(np.float64),
                              np.float64(code - 8) * scales.astype(np.float64))
        t1 = to_bf16(v)
        t2 = to_bf16((v - t1).astype(np.float32))
        assert np.array_equal(t1.astype(np.float64) + t2.astype(np.float64),
                              v.astype(np.float64)), code


def test_an_e4m3_code_becomes_bf16_by_a_shift_and_a_multiply_by_2_to_the_120():
    """The seven low bits of a code, shifted left by four, are a bf16 with the
    code's mantissa and an exponent field 120 too small (a bf16 subnormal for
    the eight subnormal codes); times 2^120 that is the code's value, which bf16
    holds exactly. The fp8 product of many rows unpacks its weights this way."""
    def e4m3(c):
        sign = -1.0 if c & 0x80 else 1.0
        e, m = (c >> 3) & 15, c & 7
        return sign * (m * 2.0 ** -9 if e == 0 else 2.0 ** (e - 7) * (1 + m / 8))
    assert bf16_bits_to_f64(0x7B80) == 2.0 ** 120
    for c in range(256):
        if (c & 0x7F) == 0x7F:
            continue                                        # the two NaN codes
        small = ((c & 0x7F) << 4) | ((c & 0x80) << 8)
        value = bf16_bits_to_f64(small) * 2.0 ** 120
        assert value == e4m3(c), c
        assert to_bf16(np.float32(value)) == np.float32(value)   # 4 bits: exact


def mma_16x8x16(a_regs, b_regs):
    """mma.sync.m16n8k16 from per-lane registers, by the fragment layout of the
    PTX manual: lane = 4 g + t holds A[g or g + 8][2t, 2t + 1 (+ 8)] and
    B[2t, 2t + 1 (+ 8)][g], and gets C[g or g + 8][2t, 2t + 1]. a_regs[lane] =
    (a0, a1, a2, a3), b_regs[lane] = (b0, b1), each a pair of values."""
    A, B = np.zeros((16, 16)), np.zeros((16, 8))
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        a0, a1, a2, a3 = a_regs[lane]
        A[g, 2 * t:2 * t + 2], A[g + 8, 2 * t:2 * t + 2] = a0, a1
        A[g, 2 * t + 8:2 * t + 10], A[g + 8, 2 * t + 8:2 * t + 10] = a2, a3
        b0, b1 = b_regs[lane]
        B[2 * t:2 * t + 2, g], B[2 * t + 8:2 * t + 10, g] = b0, b1
    return A @ B


def test_the_column_orders_of_the_quantised_tensor_core_kernels():
    """Which column of a 32-column Q4_0 group (of a 16-column fp8 step) a lane
    feeds into which k slot of the MMA is free, as long as A and B agree. The
    Q4_0 kernels pair the codes of a word as (0,4) (1,5) (2,6) (3,7), one mask
    per pair, and stage the activations in that order; the fp8 kernel pairs
    (0,2) (1,3). With the layouts restated here the sixteen rows times eight
    positions come out as the plain product."""
    rng = np.random.default_rng(9)
    # Q4_0: lane t of a row holds word t (columns 8t .. 8t + 7); two MMAs a group
    codes = rng.integers(-8, 8, (16, 32)).astype(np.float64)
    x = rng.standard_normal((8, 32))
    total = np.zeros((16, 8))
    for first in (0, 2):                          # pairs P0, P1 then P2, P3
        a_regs, b_regs = [], []
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            cols = [(8 * t + first + i, 8 * t + first + i + 4) for i in (0, 1)]
            a_regs.append((codes[g, list(cols[0])], codes[g + 8, list(cols[0])],
                           codes[g, list(cols[1])], codes[g + 8, list(cols[1])]))
            b_regs.append((x[g, list(cols[0])], x[g, list(cols[1])]))
        total += mma_16x8x16(a_regs, b_regs)
    assert np.allclose(total, codes @ x.T, rtol=0, atol=1e-12)
    # fp8: lane t holds one word (columns 4t .. 4t + 3) of a 16-column step
    w = rng.standard_normal((16, 16))
    x = rng.standard_normal((8, 16))
    a_regs, b_regs = [], []
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        even, odd = [4 * t, 4 * t + 2], [4 * t + 1, 4 * t + 3]
        a_regs.append((w[g, even], w[g + 8, even], w[g, odd], w[g + 8, odd]))
        b_regs.append((x[g, even], x[g, odd]))
    assert np.allclose(mma_16x8x16(a_regs, b_regs), w @ x.T, rtol=0, atol=1e-12)
