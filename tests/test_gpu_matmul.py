"""`a @ b` through vx_plugin_dispatch_async on a B200, against the CPU oracle
and the known answers of the reference's backend tests."""
import os

import numpy as np
import pytest

from vx_b200 import abi, ops

pytestmark = pytest.mark.gpu


def rel_frobenius(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return np.linalg.norm(got - want) / np.linalg.norm(want)


def device_matmul(a, b, bf16=False):
    ta = abi.DeviceTensor.from_host(a, bf16=bf16)
    tb = abi.DeviceTensor.from_host(b, bf16=bf16)
    tc = ops.matmul(ta, tb)
    out = tc.to_host()
    for t in (ta, tb, tc):
        t.free()
    return out


def test_roles_known_answers():
    # tests/backend/pass/gpu_matmul_roles.vx EXPECT: 38 56 83 128 9 7 10
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    b = np.arange(1, 13, dtype=np.float32).reshape(3, 4)
    c = device_matmul(a, b)
    assert [c[0, 0], c[0, 3], c[1, 0], c[1, 3]] == [38, 56, 83, 128]
    p = np.arange(1, 10, dtype=np.float32).reshape(3, 3)
    q = np.diag(np.arange(1, 4, dtype=np.float32))
    r = device_matmul(p, q)
    assert [r[0, 2], r[2, 0], r[1, 1]] == [9, 7, 10]


def test_dtypes_known_answers():
    # tests/backend/pass/gpu_matmul_dtypes.vx EXPECT: 19 50 197 4032
    a = np.array([[1, 2], [3, 4]], dtype=np.float64)
    b = np.array([[5, 6], [7, 8]], dtype=np.float64)
    c = device_matmul(a, b)
    assert (c[0, 0], c[1, 1]) == (19, 50)
    e = np.eye(64, dtype=np.float32)
    m = np.arange(64 * 64, dtype=np.float32).reshape(64, 64)
    r = device_matmul(e, m)
    assert (r[3, 5], r[63, 0]) == (197, 4032)


def test_matmul_into_buffer_known_answer():
    # tests/backend/pass/matmul_into_buffer.vx EXPECT: 3 7 3 7
    w = np.array([[1, 2], [3, 4]], dtype=np.float32)
    x = np.ones((2, 1), dtype=np.float32)
    tw, tx = abi.DeviceTensor.from_host(w), abi.DeviceTensor.from_host(x)
    ty = abi.DeviceTensor.from_host(np.full((2, 1), -1, np.float32))
    ops.matmul_into(ty, tw, tx)
    y = ty.to_host()
    assert [y[0, 0], y[1, 0]] == [3, 7]
    for t in (tw, tx, ty):
        t.free()


def test_matmul_execution_all_24():
    # benchmarks/matmul_execution.vx: 2s @ 3s over k = 4
    c = device_matmul(np.full((4, 4), 2, np.float32), np.full((4, 4), 3, np.float32))
    assert (c == 24).all()


@pytest.mark.parametrize("slot", [True, False])
def test_host_operands_slot_and_buffer(oracle, slot):
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (37, 53)).astype(np.float32)
    b = rng.uniform(-1, 1, (53, 29)).astype(np.float32)
    got = ops.matmul_host(a, b, slot=slot)
    assert rel_frobenius(got, oracle.gemm(a, b)) <= 1e-6


def test_config1_f32_1024(oracle):
    # f32 1024^3, U[-1,1), seeds 0 and 1; full C within 1e-4 rel. Frobenius.
    a = np.random.default_rng(0).uniform(-1, 1, (1024, 1024)).astype(np.float32)
    b = np.random.default_rng(1).uniform(-1, 1, (1024, 1024)).astype(np.float32)
    want = oracle.gemm(a, b, fast=True)
    got = device_matmul(a, b)
    assert rel_frobenius(got, want) <= 1e-4


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 7), (129, 130, 17),
                                   (128, 128, 16), (257, 65, 300), (64, 1, 64)])
def test_f32_ragged_shapes(oracle, m, n, k):
    rng = np.random.default_rng(m * 1000 + n * 10 + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    assert rel_frobenius(device_matmul(a, b), oracle.gemm(a, b)) <= 1e-5


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (300, 260, 128),
                                   (257, 512, 192), (128, 4096, 64)])
def test_f32_on_the_tensor_cores_is_as_good_as_the_fp32_kernel(m, n, k, monkeypatch):
    """An f32 product large enough runs as exact bf16 terms on the tensor
    cores (k a multiple of 64, n of 4). Against an f64 product its error must
    be of the size of the FP32 kernel's own, and both far inside the 1e-4 of
    the reference's check."""
    rng = np.random.default_rng(m + n + k)
    a = (rng.uniform(-1, 1, (m, k)) * np.exp(rng.uniform(-6, 6, (m, k)))).astype(np.float32)
    b = (rng.uniform(-1, 1, (k, n)) * np.exp(rng.uniform(-6, 6, (k, n)))).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    split = device_matmul(a, b)
    monkeypatch.setenv("VXB_F32_TENSOR", "0")
    plain = device_matmul(a, b)
    assert ops.kernel_status() == 0
    e_split, e_plain = rel_frobenius(split, want), rel_frobenius(plain, want)
    assert e_plain <= 2e-6 and e_split <= 2e-6, (e_split, e_plain)
    assert e_split <= 4 * e_plain + 1e-7, (e_split, e_plain)
    assert not np.array_equal(split, plain) or m * n * k < 2 ** 24


def test_f32_on_the_tensor_cores_is_exact_on_integers():
    """Integers below 2^24 are sums of three bf16 terms exactly, their products
    and sums below 2^24 are exact in f32: no tolerance."""
    rng = np.random.default_rng(77)
    a = rng.integers(-2000, 2000, (256, 256)).astype(np.float32)
    b = rng.integers(-3, 4, (256, 512)).astype(np.float32)
    want = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(device_matmul(a, b), want)


def test_strided_view_with_offset(oracle):
    # A view into a larger buffer: non-zero offset, row stride > width.
    rng = np.random.default_rng(9)
    big = rng.uniform(-1, 1, (40, 64)).astype(np.float32)
    b = rng.uniform(-1, 1, (24, 16)).astype(np.float32)
    tbig = abi.DeviceTensor.from_host(big)
    tb = abi.DeviceTensor.from_host(b)
    tc = abi.DeviceTensor.empty((32, 16), abi.F32)
    da = abi.descriptor(tbig.ptr, (32, 24), strides=(64, 1), offset=3 * 64 + 8)
    db = abi.descriptor(tb.ptr, b.shape)
    dc = abi.descriptor(tc.ptr, (32, 16))
    blob = abi.payload("k", abi=1, kind="matmul", roles="a:0,b:1,out:2",
                       outkind="buffer", topo=abi.gpu(0))
    abi.dispatch(blob, [da, db, dc], [abi.memref_tag(abi.F32, 2)] * 3)
    want = oracle.gemm(np.ascontiguousarray(big[3:35, 8:32]), b)
    assert rel_frobenius(tc.to_host(), want) <= 1e-6


def test_strided_views_on_the_tensor_core_f32_route():
    """Views large enough for the tensor-core route: A and B inside wider
    buffers at an offset, C into the middle of a wider buffer (row stride >
    width, so the partial sums go through the adding kernel)."""
    rng = np.random.default_rng(19)
    abig = rng.uniform(-1, 1, (300, 200)).astype(np.float32)
    bbig = rng.uniform(-1, 1, (140, 520)).astype(np.float32)
    cbig = np.full((260, 600), 7.0, np.float32)
    ta, tb, tc = (abi.DeviceTensor.from_host(x) for x in (abig, bbig, cbig))
    m, n, k = 256, 512, 128
    da = abi.descriptor(ta.ptr, (m, k), strides=(200, 1), offset=5 * 200 + 8)
    db = abi.descriptor(tb.ptr, (k, n), strides=(520, 1), offset=2 * 520 + 4)
    dc = abi.descriptor(tc.ptr, (m, n), strides=(600, 1), offset=600 + 12)
    blob = abi.payload("k", abi=1, kind="matmul", roles="a:0,b:1,out:2",
                       outkind="buffer", topo=abi.gpu(0))
    abi.dispatch(blob, [da, db, dc], [abi.memref_tag(abi.F32, 2)] * 3)
    got = tc.to_host()
    want = abig[5:5 + m, 8:8 + k].astype(np.float64) @ \
        bbig[2:2 + k, 4:4 + n].astype(np.float64)
    assert rel_frobenius(got[1:1 + m, 12:12 + n], want) <= 2e-6
    untouched = got.copy()
    untouched[1:1 + m, 12:12 + n] = 7.0
    assert np.all(untouched == 7.0)
    assert ops.kernel_status() == 0


def test_flat_matvec(oracle):
    rng = np.random.default_rng(3)
    w = rng.uniform(-1, 1, (300, 288)).astype(np.float32)
    x = rng.uniform(-1, 1, 288).astype(np.float32)
    got = ops.matvec_flat(w, x)
    assert np.abs(got - oracle.matvec_f32(w, x)).max() <= 1e-4


# ---- 16-bit ---------------------------------------------------------------------
def bf16_inputs(oracle, m, n, k, seed=3):
    a = np.random.default_rng(seed).uniform(-1, 1, (m, k)).astype(np.float32)
    b = np.random.default_rng(seed + 1000).uniform(-1, 1, (k, n)).astype(np.float32)
    return oracle.f32_to_bf16(a), oracle.f32_to_bf16(b)


def run_route(a16, b16, route):
    m, k = a16.shape
    n = b16.shape[1]
    ta = abi.DeviceTensor.from_host(a16, bf16=True)
    tb = abi.DeviceTensor.from_host(b16, bf16=True)
    tc = abi.DeviceTensor.empty((m, n), abi.BF16)
    ts = abi.DeviceTensor.empty((n, k), abi.BF16) if route in (2, 5) else None
    ops.gemm(ta, tb, tc, route=route, scratch=ts)
    status = ops.kernel_status()
    out = tc.to_host()
    for t in (ta, tb, tc, ts):
        if t is not None:
            t.free()
    return out, status


# 1, 2: one CTA per 128x256 tile (B as stored / transposed first); 3: the plain
# kernel; 4, 5: the same two forms on CTA pairs (256x256 tiles)
ROUTES = [int(r) for r in os.environ.get("VX_TEST_ROUTES", "3,2,1,4,5").split(",")]


@pytest.mark.parametrize("route", ROUTES)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256),
                                   (384, 768, 1024), (200, 264, 136),
                                   (2048, 2048, 2048), (2304, 1280, 512)])
def test_bf16_gemm_routes(oracle, route, m, n, k):
    a16, b16 = bf16_inputs(oracle, m, n, k)
    got, status = run_route(a16, b16, route)
    assert status == 0, "a wait in the tcgen05 kernel gave up: 0x%x" % status
    rows = np.unique(np.linspace(0, m - 1, 24).astype(np.int64))
    want = oracle.bf16_to_f32(oracle.gemm_bf16_rows(a16, b16, rows))
    err = rel_frobenius(oracle.bf16_to_f32(got[rows]), want)
    assert err <= 2e-2, err
    # f32 accumulation and one rounding: far inside the bound.
    assert err <= 4e-3, err


def test_bf16_dispatch_route_is_exact_on_small_integers(oracle):
    # The method of benchmarks/gpu_gemm/cublas_gemm.cu:22-28, 84-92: inputs are
    # small integers, so every f32 sum is exact whatever its order.
    m = n = k = 1024
    i = np.arange(m)[:, None]
    j = np.arange(k)[None, :]
    a = ((i * 3 + j * 5) % 7 - 3).astype(np.float32)
    b = ((np.arange(k)[:, None] * 2 + np.arange(n)[None, :]) % 5 - 2).astype(np.float32)
    a16, b16 = oracle.f32_to_bf16(a), oracle.f32_to_bf16(b)
    got = oracle.bf16_to_f32(device_matmul(a16, b16, bf16=True))
    assert ops.kernel_status() == 0
    for s in range(64):
        r, c = (s * 7919) % m, (s * 104729) % n
        want = oracle.gemm_bf16_entry(a16, b16, r, c)
        # the bf16 result is the exact f32 sum rounded once
        assert got[r, c] == oracle.bf16_to_f32(oracle.f32_to_bf16(np.float32(want)))


def test_bf16_pair_route_is_exact_on_small_integers(oracle):
    """The CTA-pair kernel on exact inputs: every one of the 4608 x 3072
    results must be the exact sum rounded once (which half of which tile a
    value came from cannot hide in a tolerance)."""
    m, n, k = 4608, 3072, 640       # 18 x 12 pair tiles: more than one per pair
    i = np.arange(m)[:, None]
    a = ((i * 3 + np.arange(k)[None, :] * 5) % 7 - 3).astype(np.float32)
    b = ((np.arange(k)[:, None] * 2 + np.arange(n)[None, :]) % 5 - 2).astype(np.float32)
    a16, b16 = oracle.f32_to_bf16(a), oracle.f32_to_bf16(b)
    got, status = run_route(a16, b16, 4)
    assert status == 0, "a wait in the paired kernel gave up: 0x%x" % status
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(got, oracle.f32_to_bf16(exact))


def test_f16_gemm(oracle):
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (256, 320)).astype(np.float16)
    b = rng.uniform(-1, 1, (320, 512)).astype(np.float16)
    got = device_matmul(a, b).astype(np.float32)
    assert ops.kernel_status() == 0
    want = a.astype(np.float32) @ b.astype(np.float32)
    assert rel_frobenius(got, want) <= 2e-3
