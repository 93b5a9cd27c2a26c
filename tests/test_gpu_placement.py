"""The placement, stream and image-launch entry points on a B200, called as a
compiled Vx program calls them."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from vx_b200 import abi
from vx_b200.lib import lib

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_transfer_out_and_home():
    data = np.arange(100000, dtype=np.float32)
    t = abi.DeviceTensor.from_host(data)
    assert np.array_equal(t.to_host(), data)
    t.free()


def test_transfer_async_through_pinned_staging():
    # 20 MiB: three pinned chunks; the caller may reuse its memory at once
    data = np.random.default_rng(0).integers(0, 2 ** 31, 5 * 2 ** 20, dtype=np.int32)
    keep = data.copy()
    t = abi.DeviceTensor.from_host(data, asynchronous=True)
    data[:] = 0
    assert np.array_equal(t.to_host(), keep)
    t.free()


def test_uninit_then_peer_copy_on_one_gpu():
    L = lib()
    src = abi.DeviceTensor.from_host(np.arange(4096, dtype=np.float64))
    p = L.vx_plugin_transfer_peer(src.ptr, abi.gpu(0), abi.gpu(0), src.nbytes)
    copy = abi.DeviceTensor(p, src.shape, src.elem, abi.gpu(0))
    assert np.array_equal(copy.to_host(), src.to_host())
    copy.free()
    src.free()


def test_control_opcodes_and_a_declared_topology():
    L = lib()
    assert L.vx_plugin_control(0x01, None) == 1            # INIT_DEVICE
    assert L.vx_plugin_control(0x03, None) >= 1            # GET_DEVICE_COUNT
    pair = (C.c_int32 * 2)(4242, abi.gpu(0))               # a name that hashes to 4242
    assert L.vx_plugin_control(0x04, C.addressof(pair)) == 1
    data = np.arange(64, dtype=np.float32)
    t = abi.DeviceTensor.from_host(data, topo=4242)        # lands on GPU 0
    assert np.array_equal(t.to_host(), data)
    t.free()
    topo = C.c_int32(abi.gpu(0))
    for opcode in (0x05, 0x07):
        assert L.vx_plugin_control(opcode, C.addressof(topo)) == 1


def test_arrival_counts_are_kept_per_site():
    L = lib()
    site = C.create_string_buffer(b"site")
    zeros = (C.c_uint32 * 4)()
    a = L.vx_plugin_arrivals_take(site, 16, zeros, abi.gpu(0), 1)
    L.vx_plugin_arrivals_give(site, a, 16, abi.gpu(0))
    b = L.vx_plugin_arrivals_take(site, 16, zeros, abi.gpu(0), 1)
    assert a == b                                           # the kept counter
    c = L.vx_plugin_arrivals_take(site, 16, zeros, abi.gpu(0), 1)
    assert c != b                                           # none kept: a new one
    L.vx_plugin_arrivals_give(site, b, 16, abi.gpu(0))
    L.vx_plugin_arrivals_give(site, c, 16, abi.gpu(0))      # spare is freed


def test_caller_stream_and_graph_recording():
    """A GEMM on device tensors records into a CUDA graph on the caller's
    stream (docs/lang/abi.md 3.6) and replays."""
    import torch
    from vx_b200 import ops
    a = np.random.default_rng(1).uniform(-1, 1, (128, 64)).astype(np.float32)
    b = np.random.default_rng(2).uniform(-1, 1, (64, 96)).astype(np.float32)
    ta, tb = abi.DeviceTensor.from_host(a), abi.DeviceTensor.from_host(b)
    tc = abi.DeviceTensor.from_host(np.zeros((128, 96), np.float32))
    stream = torch.cuda.Stream()
    L = lib()
    L.vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    try:
        assert L.vx_cuda_get_stream() == stream.cuda_stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            ops.matmul_into(tc, ta, tb)
        graph.replay()
        stream.synchronize()
    finally:
        L.vx_cuda_set_stream(None)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(tc.to_host() - want).max() <= 1e-4


PTX_KERNEL = r"""
extern "C" __global__ void vx_npu_kernel_7(
    float *a_alloc, float *a, long long a_off, long long a_n, long long a_s,
    float *y_alloc, float *y, long long y_off, long long y_n, long long y_s,
    float alpha, int n)
{
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += gridDim.x * blockDim.x)
    y[y_off + i * y_s] = alpha * a[a_off + i * a_s];
}
"""


def test_a_compiler_style_ptx_image_is_loaded_and_launched(tmp_path):
    """A region that is not a matmul carries PTX text in `image=`; two rank-1
    memrefs are 2 x 5 parameters, then the scalars; `launch=` gives the trip
    count of the grid-strided loop."""
    src = tmp_path / "k.cu"
    src.write_text(PTX_KERNEL)
    ptx = tmp_path / "k.ptx"
    subprocess.run(["nvcc", "-ptx", "-arch=sm_100a", str(src), "-o", str(ptx)],
                   check=True)
    text = ptx.read_text()
    n = 1000
    a = np.arange(n, dtype=np.float32)
    ta = abi.DeviceTensor.from_host(a)
    ty = abi.DeviceTensor.from_host(np.zeros(n, np.float32))
    blob = abi.payload("vx_npu_kernel_7", abi=1, topo=abi.gpu(0),
                       launch=n, format="ptx", image=text)
    da, dy = abi.descriptor(ta.ptr, (n,)), abi.descriptor(ty.ptr, (n,))
    alpha, count = C.c_float(2.5), C.c_int32(n)
    tags = [abi.memref_tag(abi.F32, 1), abi.memref_tag(abi.F32, 1), 6, 4]
    for _ in range(2):                      # the second call hits the cache
        abi.dispatch(blob, [da, dy, alpha, count], tags)
    assert np.array_equal(ty.to_host(), a * np.float32(2.5))
