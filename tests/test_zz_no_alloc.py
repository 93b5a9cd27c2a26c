"""The attention entry point that allocates nothing
(vx_b200_attention_decode_static): for hosts that cannot call cudaMalloc --
a process whose own pool took all device memory at start-up, or a loop that
cannot take the device-wide wait of an allocation -- the scratch is a fixed
array inside the library. Checked against vx_nn_attention, which takes its
scratch from the caller, on two calls in a row (the array keeps the first
call's contents, and the counters must be back at zero)."""
import numpy as np
import pytest

from vx_b200 import abi, ops
from vx_b200.lib import lib

pytestmark = pytest.mark.gpu


def both(oracle, qh, kvh, hd, pos, max_seq, seed):
    q = oracle.random_f32(qh * hd, seed, 2.0).reshape(qh, hd)
    kc = oracle.random_f32(max_seq * kvh * hd, seed + 1, 2.0).reshape(max_seq, kvh, hd)
    vc = oracle.random_f32(max_seq * kvh * hd, seed + 2, 1.0).reshape(max_seq, kvh, hd)
    tq, tk, tv = (abi.DeviceTensor.from_host(t) for t in (q, kc, vc))
    part = abi.DeviceTensor.empty(
        ops.nn_attention_scratch_shape(max_seq, qh, kvh, hd), abi.F32)
    want = abi.DeviceTensor.empty((qh, hd), abi.F32)
    ops.nn_attention(want, part, tq, tk, tv, pos, qh, kvh, hd)
    got = abi.DeviceTensor.empty((qh, hd), abi.F32)
    rc = lib().vx_b200_attention_decode_static(got.ptr, tq.ptr, tk.ptr, tv.ptr,
                                               pos, qh, kvh, hd)
    assert rc == 0, lib().vx_b200_last_error()
    g, w = got.to_host(), want.to_host()
    for t in (tq, tk, tv, part, want, got):
        t.free()
    return g, w, oracle.attention_f64(q, kc, vc, pos)


def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(oracle):
    for qh, kvh, hd, pos, max_seq, seed in [(28, 4, 128, 300, 400, 61),
                                            (32, 2, 64, 655, 704, 71)]:
        got, want, exact = both(oracle, qh, kvh, hd, pos, max_seq, seed)
        bound = 1e-5 * np.abs(exact).max()
        assert np.abs(got - want).max() <= bound
        assert np.abs(got - exact).max() <= bound


def test_a_size_beyond_the_static_scratch_is_refused():
    # 256 heads of 128 at position 4095 need 256 * 64 * 130 floats > 2^19
    rc = lib().vx_b200_attention_decode_static(None, None, None, None, 4095, 256,
                                               256, 128)
    assert rc == -1
    assert b"static scratch holds" in lib().vx_b200_last_error()
