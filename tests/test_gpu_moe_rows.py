"""The mixture-of-experts kernels for many positions, and the quantised products
of many rows that share their tensor-core kernel.

The pairs grouped by expert (nn_moe_group*, stdlib/std/nn.vx:1056-1294) bit-exact
against the plain stable sort on the reference's own cases (tests/optimizations/
pass/std_nn_moe_group_sorts_pairs_by_expert.vx). The `_rows` router and Q4_0
projections on the sizes of apple_gpu_kernels_for_n_positions_match_one_position.vx
(5 positions; 16 experts, 4 a position): every row bit for bit the one-position
kernel's, and within the reference's criterion of f64 loops. The grouped expert
projections (vx_b200_moe_*_grouped) and the Q4_0 / fp8 products of many rows
(vx_b200_gemm_q4, vx_b200_gemm_fp8) against f64 loops by the same criterion, max
|got - want| <= 1e-5 * max |want|."""
import numpy as np
import pytest

from vx_b200 import abi, ops

pytestmark = pytest.mark.gpu


def dev(a, bf16=False):
    return abi.DeviceTensor.from_host(a, bf16=bf16)


def empty(shape, elem=abi.I32):
    return abi.DeviceTensor.empty(shape, elem)


def close(got, want, tol=1e-5):
    want = np.asarray(want, np.float64)
    worst = np.abs(np.asarray(got, np.float64) - want).max()
    assert worst <= tol * np.abs(want).max(), (worst, np.abs(want).max())


def group_on_gpu(ids, experts, align, room=None, in_steps=False, wide=0):
    """All five outputs; `wide` extra columns in counts and base."""
    n = ids.size
    room = n + experts * (align - 1) if room is None else room
    tiles = (room + align - 1) // align
    blocks = max((n + 255) // 256, 1)
    fill = np.full
    order = dev(fill(max(room, 1), -5, np.int32)).view(0, (room,))
    counts = dev(fill((blocks, experts + wide), -5, np.int32))
    base = dev(fill((blocks, experts + wide), -5, np.int32))
    starts = dev(fill(experts + 1, -5, np.int32))
    tile_expert = dev(fill(max(tiles, 1), -5, np.int32)).view(0, (tiles,))
    t_ids = dev(ids if n else np.zeros(1, np.int32)).view(0, (n,))
    if in_steps:
        ops.nn_moe_group_count(counts, t_ids, n, experts)
        ops.nn_moe_group_offsets(base, starts, tile_expert, order, counts, n, experts,
                                 align)
        ops.nn_moe_group_place(order, t_ids, base, n)
    else:
        ops.nn_moe_group(order, counts, base, starts, tile_expert, t_ids, experts,
                         align)
    live = (n + 255) // 256
    return dict(order=order.to_host(), starts=starts.to_host(),
                tile_expert=tile_expert.to_host(),
                counts=counts.to_host()[:live, :experts],
                base=base.to_host()[:live, :experts])


@pytest.mark.parametrize("in_steps", [False, True])
def test_moe_group_on_the_reference_cases(oracle, in_steps):
    for name, ids, experts, align in oracle.moe_group_reference_cases():
        want = oracle.moe_group(ids, experts, align)
        got = group_on_gpu(ids, experts, align, in_steps=in_steps)
        for key in want:
            assert np.array_equal(got[key], want[key]), (name, key)
    assert ops.kernel_status() == 0


def test_moe_group_edges(oracle):
    rng = np.random.default_rng(5)
    cases = [(np.zeros(0, np.int32), 3, 4, None),          # no pair at all
             (np.array([2, 2, 2], np.int32), 3, 4, None),  # empty groups in front
             (np.arange(256, dtype=np.int32) % 7, 7, 8, None),   # one full block
             (np.arange(257, dtype=np.int32) % 1024, 1024, 1, None),
             # a prompt's worth: 4096 positions x 2 of 8 experts, tiles of 128
             (rng.integers(0, 8, 8192).astype(np.int32), 8, 128, None),
             # more room than needed: the rest holds n + i and tiles of -1
             (rng.integers(0, 60, 3000).astype(np.int32), 64, 16, 3000 + 64 * 15 + 100),
             # every pair at the last of 1024 experts
             (np.full(1500, 1023, np.int32), 1024, 4, None)]
    for ids, experts, align, room in cases:
        want = oracle.moe_group(ids, experts, align, room)
        got = group_on_gpu(ids, experts, align, room, wide=3)
        for key in want:
            assert np.array_equal(got[key], want[key]), (ids.size, experts, align, key)
    assert ops.kernel_status() == 0


def test_moe_group_reports_an_id_that_names_no_expert(oracle):
    ids = np.array([0, 1, 9, 2, -1, 1], np.int32)
    got = group_on_gpu(ids, 3, 1)
    assert ops.kernel_status() == 0x6E
    assert ops.kernel_status() == 0            # reported once
    # the other pairs are grouped as if the two were not there
    assert list(got["counts"][0]) == [1, 2, 1]
    assert list(got["order"][:4]) == [0, 1, 5, 3]


def router_logits(oracle, n, experts):
    """Position t favours the experts near 3 t, so neighbours share some
    (the reference test's router, :243-250)."""
    e = np.arange(experts)[None, :]
    t = np.arange(n)[:, None]
    noise = oracle.random_f32(n * experts, 31, 0.005).reshape(n, experts)
    return (-0.1 * (e - 3 * t) ** 2 + noise).astype(np.float32)


def test_top_k_rows(oracle):
    n, experts, k = 5, 16, 4
    logits = router_logits(oracle, n, experts)
    wide = np.zeros((n, experts + 3), np.float32)      # a pitch above `count`
    wide[:, :experts] = logits
    tid, tw = empty((n, k + 1)), empty((n, k + 2), abi.F32)
    ops.nn_top_k_rows(tid, tw, dev(wide), n, experts, k)
    ids, weights = tid.to_host()[:, :k], tw.to_host()[:, :k]
    for t in range(n):
        one_i, one_w = empty((k,)), empty((k,), abi.F32)
        ops.nn_top_k(one_i, one_w, dev(logits[t]), experts, k)
        assert np.array_equal(ids[t], one_i.to_host()), t
        assert np.array_equal(weights[t], one_w.to_host()), t
        want_i, want_w = oracle.nn_top_k(logits[t], k)
        assert np.array_equal(ids[t], want_i), t
        close(weights[t], want_w, 2e-6)
    # 256 experts, all of them kept, and a tie
    logits = oracle.random_f32(3 * 256, 32, 2.0).reshape(3, 256)
    logits[1, 200] = logits[1, 17] = 7.0
    tid, tw = empty((3, 256)), empty((3, 256), abi.F32)
    ops.nn_top_k_rows(tid, tw, dev(logits), 3, 256, 256)
    for t in range(3):
        want_i, want_w = oracle.nn_top_k(logits[t], 256)
        assert np.array_equal(tid.to_host()[t], want_i), t
        close(tw.to_host()[t], want_w, 2e-6)
    assert list(tid.to_host()[1, :2]) == [17, 200]


def test_q4_rows_projections_match_one_position_bit_for_bit(oracle):
    n, rows, cols, heads, hd = 5, 64, 256, 4, 64
    w, s = oracle.quant_inputs("q4", rows, cols, 41)
    tw, ts = dev(w), dev(s)
    x = oracle.random_f32(n * cols, 42, 1.0).reshape(n, heads, hd)
    y0 = oracle.random_f32(n * rows, 43, 1.0).reshape(n, rows)
    ty = dev(y0)
    ops.nn_matvec_q4_heads_add_rows(ty, tw, ts, dev(x), n, rows, heads, hd)
    got = ty.to_host()
    for t in range(n):
        one = dev(y0[t])
        ops.nn_matvec_quant_heads_add("q4", one, tw, ts, dev(x[t]), rows, heads, hd)
        assert np.array_equal(got[t], one.to_host()), t
        want = y0[t] + oracle.quant_dot_f64("q4", w, s, x[t].reshape(-1), rows, cols)
        close(got[t], want)
    # Q, K and V of 4 + 2 + 2 heads with a bias
    qh, kvh = 4, 2
    allrows = (qh + 2 * kvh) * hd
    wq, sq = oracle.quant_inputs("q4", allrows, cols, 44)
    bias = oracle.f32_to_bf16(oracle.random_f32(allrows, 45, 0.5))
    twq, tsq, tb = dev(wq), dev(sq), dev(bias, True)
    xr = x.reshape(n, cols)
    tq, tk, tv = (empty((n, h, hd), abi.F32) for h in (qh, kvh, kvh))
    ops.nn_qkv_q4_rows(tq, tk, tv, twq, tsq, tb, dev(xr), n, qh, kvh, hd, cols)
    gq, gk, gv = tq.to_host(), tk.to_host(), tv.to_host()
    for t in range(n):
        q1, k1, v1 = (empty((h, hd), abi.F32) for h in (qh, kvh, kvh))
        ops.nn_qkv_quant("q4", q1, k1, v1, twq, tsq, tb, dev(xr[t]), qh, kvh, hd, cols)
        assert np.array_equal(gq[t], q1.to_host()), t
        assert np.array_equal(gk[t], k1.to_host()), t
        assert np.array_equal(gv[t], v1.to_host()), t
        want = oracle.quant_dot_f64("q4", wq, sq, xr[t], allrows, cols) \
            + oracle.bf16_to_f32(bias)
        close(np.concatenate([gq[t].ravel(), gk[t].ravel(), gv[t].ravel()]), want)
    assert ops.kernel_status() == 0


def test_experts_of_n_positions(oracle):
    """nn_top_k_rows -> nn_moe_swiglu_q4_rows -> nn_moe_down_q4_add_rows against
    the one-position kernels (bit for bit) and f64 loops; the grouping of the
    same ids says how many experts the 5 positions use."""
    n, experts, k, inter, cols = 5, 16, 4, 64, 256
    logits = router_logits(oracle, n, experts)
    tid, tw = empty((n, k)), empty((n, k), abi.F32)
    ops.nn_top_k_rows(tid, tw, dev(logits), n, experts, k)
    ids, weights = tid.to_host(), tw.to_host()
    gu, gu_s = oracle.quant_inputs("q4", experts * 2 * inter, cols, 51)
    dn, dn_s = oracle.quant_inputs("q4", experts * cols, inter, 53)
    t_gu, t_gus, t_dn, t_dns = dev(gu), dev(gu_s), dev(dn), dev(dn_s)
    x = oracle.random_f32(n * cols, 55, 1.0).reshape(n, cols)
    y0 = oracle.random_f32(n * cols, 56, 1.0).reshape(n, cols)
    mid = empty((n * k, inter), abi.F32)
    ops.nn_moe_swiglu_q4_rows(mid, t_gu, t_gus, tid, dev(x), n, k, inter, cols, experts)
    ty = dev(y0)
    ops.nn_moe_down_q4_add_rows(ty, t_dn, t_dns, tid, tw, mid, n, k, cols, inter,
                                experts)
    got_mid, got_y = mid.to_host(), ty.to_host()
    for t in range(n):
        m1 = empty((k, inter), abi.F32)
        ops.nn_moe_swiglu(m1, t_gu, dev(ids[t]), dev(x[t]), k, inter, cols, experts,
                          scales=t_gus)
        y1 = dev(y0[t])
        ops.nn_moe_down_add(y1, t_dn, dev(ids[t]), dev(weights[t]), m1, k, cols, inter,
                            experts, scales=t_dns)
        assert np.array_equal(got_mid[t * k:(t + 1) * k], m1.to_host()), t
        assert np.array_equal(got_y[t], y1.to_host()), t
        gate_up = oracle.quant_dot_f64("q4", gu, gu_s, x[t], experts * 2 * inter, cols)
        want_y = y0[t].astype(np.float64)
        for e in range(k):
            g = gate_up[ids[t, e] * 2 * inter:ids[t, e] * 2 * inter + inter]
            u = gate_up[ids[t, e] * 2 * inter + inter:(ids[t, e] + 1) * 2 * inter]
            close(got_mid[t * k + e], g / (1.0 + np.exp(-g)) * u)
            down = oracle.quant_dot_f64("q4", dn, dn_s, got_mid[t * k + e],
                                        experts * cols, inter)
            want_y += float(weights[t, e]) * down[ids[t, e] * cols:(ids[t, e] + 1) * cols]
        close(got_y[t], want_y)
    # the same pairs grouped by expert, in tiles of 8
    flat = ids.reshape(-1)
    want = oracle.moe_group(flat, experts, 8)
    got = group_on_gpu(flat, experts, 8)
    for key in want:
        assert np.array_equal(got[key], want[key]), key
    used = np.count_nonzero(np.diff(got["starts"]))
    assert used == np.unique(flat).size and 4 < used < 16
    assert ops.kernel_status() == 0


def grouped_layer(oracle, n, experts, k, inter, hidden, seed, align):
    """Router -> grouping in tiles of `align` -> the two expert projections on the
    tensor cores; returns what the f64 check needs."""
    logits = oracle.random_f32(n * experts, seed, 2.0).reshape(n, experts)
    tid, tw = empty((n, k)), empty((n, k), abi.F32)
    ops.nn_top_k_rows(tid, tw, dev(logits), n, experts, k)
    ids, weights = tid.to_host(), tw.to_host()
    gu, gu_s = oracle.quant_inputs("q4", experts * 2 * inter, hidden, seed + 1)
    dn, dn_s = oracle.quant_inputs("q4", experts * hidden, inter, seed + 3)
    x = oracle.random_f32(n * hidden, seed + 5, 1.0).reshape(n, hidden)
    y0 = oracle.random_f32(n * hidden, seed + 6, 1.0).reshape(n, hidden)
    pairs = n * k
    room = pairs + experts * (align - 1)
    tiles = (room + align - 1) // align
    blocks = (pairs + 255) // 256
    order, tile_expert = empty((room,)), empty((tiles,))
    ops.nn_moe_group(order, empty((blocks, experts)), empty((blocks, experts)),
                     empty((experts + 1,)), tile_expert, tid.view(0, (pairs,)), experts,
                     align)
    t_gu, t_gus, t_dn, t_dns = dev(gu), dev(gu_s), dev(dn), dev(dn_s)
    mid = dev(np.full((pairs, inter), np.nan, np.float32))
    ops.moe_swiglu_q4_grouped(mid, t_gu, t_gus, order, tile_expert, align, dev(x), n, k,
                              inter, hidden, experts)
    ty = dev(y0)
    scratch = dev(np.full((pairs, hidden), np.nan, np.float32))
    ops.moe_down_q4_add_grouped(ty, t_dn, t_dns, order, tile_expert, align,
                                tw.view(0, (pairs,)), mid, scratch, n, k, hidden, inter,
                                experts)
    return dict(ids=ids, weights=weights, gu=gu, gu_s=gu_s, dn=dn, dn_s=dn_s, x=x, y0=y0,
                mid=mid.to_host(), y=ty.to_host(), dev=(t_gu, t_gus, t_dn, t_dns, tid, tw))


@pytest.mark.parametrize("align", [8, 16])
@pytest.mark.parametrize("n,experts,k,inter,hidden", [
    (5, 16, 4, 64, 256),        # the reference test's sizes
    (40, 8, 2, 352, 1056),      # two column chunks, the second of 32 columns
    (24, 8, 2, 128, 1408),      # columns in steps of 128; 1408 = 1024 + 384
    (3, 4, 1, 32, 32)])         # one group of columns, tiles mostly padding
def test_grouped_experts_against_f64_loops(oracle, n, experts, k, inter, hidden, align):
    r = grouped_layer(oracle, n, experts, k, inter, hidden, 61, align)
    ids, weights = r["ids"], r["weights"]
    for t in range(n):
        gate_up = oracle.quant_dot_f64("q4", r["gu"], r["gu_s"], r["x"][t],
                                       experts * 2 * inter, hidden)
        want_y = r["y0"][t].astype(np.float64)
        for e in range(k):
            at = ids[t, e] * 2 * inter
            g, u = gate_up[at:at + inter], gate_up[at + inter:at + 2 * inter]
            close(r["mid"][t * k + e], g / (1.0 + np.exp(-g)) * u)
            down = oracle.quant_dot_f64("q4", r["dn"], r["dn_s"], r["mid"][t * k + e],
                                        experts * hidden, inter)
            want_y += float(weights[t, e]) * down[ids[t, e] * hidden:
                                                  (ids[t, e] + 1) * hidden]
        close(r["y"][t], want_y)
    # and next to the position-by-position exports, which sum in another order
    t_gu, t_gus, t_dn, t_dns, tid, tw = r["dev"]
    mid_rows = empty((n * k, inter), abi.F32)
    ops.nn_moe_swiglu_q4_rows(mid_rows, t_gu, t_gus, tid, dev(r["x"]), n, k, inter, hidden,
                              experts)
    close(r["mid"].ravel(), mid_rows.to_host().ravel(), 2e-5)
    assert ops.kernel_status() == 0


@pytest.mark.parametrize("align", [8, 16])
def test_grouped_down_projection_with_a_last_tile_of_eight_rows(oracle, align):
    """40 output rows: two 16-row tiles and a half one."""
    n, experts, k, rows, cols = 9, 3, 2, 40, 96
    ids = np.array([[(t + e) % experts for e in range(k)] for t in range(n)], np.int32)
    weights = (np.float32(0.3) + oracle.random_f32(n * k, 71, 0.2)).reshape(n, k)
    dn, dn_s = oracle.quant_inputs("q4", experts * rows, cols, 72)
    h = oracle.random_f32(n * k * cols, 73, 1.0).reshape(n * k, cols)
    y0 = oracle.random_f32(n * rows, 74, 1.0).reshape(n, rows)
    pairs, room = n * k, n * k + experts * (align - 1)
    tiles = (room + align - 1) // align
    order, tile_expert = empty((room,)), empty((tiles,))
    ops.nn_moe_group(order, empty((1, experts)), empty((1, experts)),
                     empty((experts + 1,)), tile_expert, dev(ids).view(0, (pairs,)),
                     experts, align)
    ty = dev(y0)
    ops.moe_down_q4_add_grouped(ty, dev(dn), dev(dn_s), order, tile_expert, align,
                                dev(weights).view(0, (pairs,)), dev(h),
                                empty((pairs, rows), abi.F32), n, k, rows, cols, experts)
    got = ty.to_host()
    for t in range(n):
        want = y0[t].astype(np.float64)
        for e in range(k):
            down = oracle.quant_dot_f64("q4", dn, dn_s, h[t * k + e], experts * rows, cols)
            want += float(weights[t, e]) * down[ids[t, e] * rows:(ids[t, e] + 1) * rows]
        close(got[t], want)
    assert ops.kernel_status() == 0


@pytest.mark.parametrize("n,rows,cols", [(5, 64, 256), (37, 296, 896), (512, 128, 4096),
                                         (1, 8, 32)])
def test_q4_product_of_many_rows_on_the_tensor_cores(oracle, n, rows, cols):
    """vx_b200_gemm_q4 against f64 loops, and beside vx_nn_matvec_q4_rows."""
    w, s = oracle.quant_inputs("q4", rows, cols, 81)
    x = oracle.random_f32(n * cols, 82, 1.0).reshape(n, cols)
    tw, ts, tx = dev(w), dev(s), dev(x)
    ty = dev(np.full((n, rows), np.nan, np.float32))
    ops.gemm_q4(ty, tw, ts, tx, n, rows, cols)
    got = ty.to_host()
    for t in range(0, n, max(1, n // 7)):
        close(got[t], oracle.quant_dot_f64("q4", w, s, x[t], rows, cols))
    other = empty((n, rows), abi.F32)
    ops.nn_matvec_q4_rows(other, tw, ts, tx, n, rows, cols)
    close(got.ravel(), other.to_host().ravel(), 2e-5)
    assert ops.kernel_status() == 0


@pytest.mark.parametrize("n,rows,cols", [(5, 64, 256), (37, 296, 896), (300, 128, 4096),
                                         (1, 4, 128), (16, 20, 640)])
def test_fp8_product_of_many_rows_on_the_tensor_cores(oracle, n, rows, cols):
    """vx_b200_gemm_fp8 against f64 loops over the definition of the format,
    and beside the one-position kernel run row by row."""
    w, s = oracle.quant_inputs("fp8", rows, cols, 91)
    x = oracle.random_f32(n * cols, 92, 1.0).reshape(n, cols)
    tw, ts = dev(w), dev(s)
    ty = dev(np.full((n, rows), np.nan, np.float32))
    ops.gemm_fp8(ty, tw, ts, dev(x), n, rows, cols)
    got = ty.to_host()
    for t in range(0, n, max(1, n // 7)):
        close(got[t], oracle.quant_dot_f64("fp8", w, s, x[t], rows, cols))
        one = empty((rows,), abi.F32)
        ops.nn_matvec_quant("fp8", one, tw, ts, dev(x[t]), rows, cols)
        close(got[t], one.to_host(), 2e-5)
    assert ops.kernel_status() == 0


def test_fp8_product_unpacks_every_code(oracle):
    """A matrix whose first row block holds every e4m3 code but the two NaNs,
    subnormal codes among them, against a unit vector per column: exact."""
    rows, cols = 4, 256
    codes = np.array([c for c in range(256) if (c & 0x7f) != 0x7f] + [0, 0], np.uint8)
    w = np.tile(codes, rows).reshape(rows, cols)
    w[1] = w[1][::-1]
    words = np.ascontiguousarray(w).view(np.uint32).reshape(-1)
    s = np.array([0.5, 2.0], np.float32)                 # the two column blocks
    x = np.eye(cols, dtype=np.float32)
    ty = dev(np.full((cols, rows), np.nan, np.float32))
    ops.gemm_fp8(ty, dev(words), dev(s), dev(x), cols, rows, cols)
    got = ty.to_host().astype(np.float64)
    for j in range(0, cols, 5):
        want = oracle.quant_dot_f64("fp8", words, s, x[j], rows, cols)
        assert np.array_equal(got[j], want), j
