"""The attention entry point that allocates nothing
(vx_b200_attention_decode_static): for hosts that cannot call cudaMalloc --
a process whose own pool took all device memory at start-up, or a loop that
cannot take the device-wide wait of an allocation -- the scratch of the split
attention kernel (partial results per block of positions, one counter per head
tile) is a fixed array inside the library. Checked against vx_nn_attention,
which takes its scratch from the caller, on calls in a row at different
positions: the array keeps the last call's partials, and a counter that a
launch left non-zero would make the next launch merge too early or never."""
import numpy as np
import pytest

from vx_b200 import abi, ops
from vx_b200.lib import lib

pytestmark = pytest.mark.gpu


class Case:
    def __init__(self, oracle, qh, kvh, hd, max_seq, seed):
        self.oracle, self.dims = oracle, (qh, kvh, hd)
        self.q = oracle.random_f32(qh * hd, seed, 2.0).reshape(qh, hd)
        self.kc = oracle.random_f32(max_seq * kvh * hd, seed + 1, 2.0) \
            .reshape(max_seq, kvh, hd)
        self.vc = oracle.random_f32(max_seq * kvh * hd, seed + 2, 1.0) \
            .reshape(max_seq, kvh, hd)
        self.tq, self.tk, self.tv = (abi.DeviceTensor.from_host(t)
                                     for t in (self.q, self.kc, self.vc))
        self.part = abi.DeviceTensor.empty(
            ops.nn_attention_scratch_shape(max_seq, qh, kvh, hd), abi.F32)
        self.want = abi.DeviceTensor.empty((qh, hd), abi.F32)
        self.got = abi.DeviceTensor.empty((qh, hd), abi.F32)

    def check(self, pos, reference_kernel):
        qh, kvh, hd = self.dims
        before = lib().vx_b200_attention_kernel(reference_kernel)
        ops.nn_attention(self.want, self.part, self.tq, self.tk, self.tv, pos,
                         qh, kvh, hd)
        lib().vx_b200_attention_kernel(before)
        rc = lib().vx_b200_attention_decode_static(
            self.got.ptr, self.tq.ptr, self.tk.ptr, self.tv.ptr, pos, qh, kvh, hd)
        assert rc == 0, lib().vx_b200_last_error()
        got, want = self.got.to_host(), self.want.to_host()
        exact = self.oracle.attention_f64(self.q, self.kc, self.vc, pos)
        bound = 1e-5 * np.abs(exact).max()
        assert np.abs(got - want).max() <= bound, pos
        assert np.abs(got - exact).max() <= bound, pos
        return got, want

    def free(self):
        for t in (self.tq, self.tk, self.tv, self.part, self.want, self.got):
            t.free()


def test_calls_in_a_row_match_the_entry_point_with_caller_scratch(oracle):
    """Two shapes; for each, calls back to back at positions on both sides of
    640 (where the run length goes from 32 to 64) and with more and fewer
    parts than the call before. Against the default (cluster) kernel the
    results agree within the tolerance of the operator tests; against the
    split kernel run with caller scratch they are the same bits."""
    for qh, kvh, hd, max_seq, seed, positions in [
            (28, 4, 128, 704, 61, (300, 655, 17, 300)),
            (32, 2, 64, 704, 71, (655, 0, 639, 640))]:
        case = Case(oracle, qh, kvh, hd, max_seq, seed)
        for pos in positions:
            case.check(pos, 1)
            got, want = case.check(pos, 2)
            assert np.array_equal(got, want), pos
        case.free()


def test_a_size_beyond_the_static_scratch_is_refused():
    # 256 heads of 128 at position 4095 need 256 * 64 * 130 floats > 2^19
    rc = lib().vx_b200_attention_decode_static(None, None, None, None, 4095, 256,
                                               256, 128)
    assert rc == -1
    assert b"static scratch holds" in lib().vx_b200_last_error()
    rc = lib().vx_b200_attention_decode_static(None, None, None, None, 16384, 1,
                                               1, 64)
    assert rc == -1
