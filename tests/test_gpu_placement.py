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


# ---- the rest of the image launcher: shapes from launch values, more than
# ---- 48 KiB of shared memory, the assert flag, a launch inside a recording,
# ---- and a TMA copy through a map from vx_plugin_tensor_map
LAUNCHER_KERNELS = r"""
#include <stdint.h>
extern "C" __global__ void vx_shape_kernel(
    int *o_alloc, int *o, long long o_off, long long o_n, long long o_s, int tag)
{
  // one value per thread: which block and thread wrote it, and the grid seen
  const int i = blockIdx.y * gridDim.x * blockDim.x + blockIdx.x * blockDim.x
                + threadIdx.x;
  if (i < o_n)
    o[o_off + i * o_s] = tag + 1000 * (int)gridDim.y + (int)blockDim.x;
}

extern "C" __global__ void vx_big_shared_kernel(
    float *a_alloc, float *a, long long a_off, long long a_n, long long a_s,
    float *y_alloc, float *y, long long y_off, long long y_n, long long y_s)
{
  extern __shared__ float stage[];            // 64 KiB: 16384 floats
  for (int i = threadIdx.x; i < 16384; i += blockDim.x)
    stage[i] = a[a_off + i];
  __syncthreads();
  for (int i = threadIdx.x; i < 16384; i += blockDim.x)
    y[y_off + i] = stage[16383 - i];
}

// What the compiler emits for `assert(x[i] >= 0)` with assert_flag=1: no trap;
// the kernel sets the flag and goes on.
extern "C" __global__ void vx_assert_kernel(
    float *x_alloc, float *x, long long x_off, long long x_n, long long x_s,
    int *failed)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < x_n && !(x[x_off + i * x_s] >= 0.0f))
    *failed = 1;
}

// One 8 x 16 box of f32 through a tensor map in device memory (the form
// lanes::copy_async compiles to): a plain tiled load, no multicast. The wait
// is bounded; on expiry status[0] says so and nothing is copied out.
extern "C" __global__ void vx_tma_kernel(
    float *o_alloc, float *o, long long o_off, long long o_n, long long o_s,
    int *s_alloc, int *status, long long s_off, long long s_n, long long s_s,
    long long map, int x, int y)
{
  __shared__ __attribute__((aligned(128))) float tile[8 * 16];
  __shared__ __attribute__((aligned(8))) uint64_t bar;
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(&bar);
  const uint32_t tile_a = (uint32_t)__cvta_generic_to_shared(tile);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_a));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(bar_a), "r"(8 * 16 * 4) : "memory");
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::"
                 "complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(tile_a), "l"(map), "r"(x), "r"(y), "r"(bar_a) : "memory");
  }
  bool landed = false;
  for (int spin = 0; spin < (1 << 22) && !landed; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar_a), "r"(0) : "memory");
    landed = done != 0;
  }
  if (!landed) {
    if (threadIdx.x == 0)
      status[s_off] = 1;
    return;
  }
  for (int i = threadIdx.x; i < 8 * 16; i += blockDim.x)
    o[o_off + i] = tile[i];
}
"""


@pytest.fixture(scope="module")
def launcher_ptx(tmp_path_factory):
    d = tmp_path_factory.mktemp("ptx")
    src = d / "launcher.cu"
    src.write_text(LAUNCHER_KERNELS)
    out = d / "launcher.ptx"
    subprocess.run(["nvcc", "-ptx", "-arch=sm_100a", str(src), "-o", str(out)],
                   check=True)
    return out.read_text()


def test_grid_and_block_from_launch_values(launcher_ptx):
    """`grid=$0,$1` and `block=$2`: the sizes are i32 launch values that sit
    after the kernel's arguments (runtime/vx_kernel_launch.h:395-484)."""
    gx, gy, threads = 5, 3, 64
    n = gx * gy * threads
    out = abi.DeviceTensor.from_host(np.zeros(n, np.int32))
    blob = abi.payload("vx_shape_kernel", abi=1, topo=abi.gpu(0), grid="$0,$1",
                       block="$2", format="ptx", image=launcher_ptx)
    tags = [abi.memref_tag(abi.I32, 1), abi.I32_KIND]
    abi.dispatch(blob, [abi.descriptor(out.ptr, (n,)), C.c_int32(7)], tags,
                 launch_values=(gx, gy, threads))
    assert (out.to_host() == 7 + 1000 * gy + threads).all()
    # fixed numbers in the shape text work the same way
    out2 = abi.DeviceTensor.from_host(np.zeros(n, np.int32))
    blob = abi.payload("vx_shape_kernel", abi=1, topo=abi.gpu(0), grid="5,3",
                       block="64", format="ptx", image=launcher_ptx)
    abi.dispatch(blob, [abi.descriptor(out2.ptr, (n,)), C.c_int32(9)], tags)
    assert (out2.to_host() == 9 + 1000 * gy + threads).all()
    out.free()
    out2.free()


def test_more_than_48_kib_of_shared_memory(launcher_ptx):
    """`shared=65536`: the launcher opts the kernel in before its first launch
    (runtime/cuda_dispatch.cpp:1484-1502)."""
    a = np.arange(16384, dtype=np.float32)
    ta = abi.DeviceTensor.from_host(a)
    ty = abi.DeviceTensor.from_host(np.zeros(16384, np.float32))
    blob = abi.payload("vx_big_shared_kernel", abi=1, topo=abi.gpu(0), grid="1",
                       block="256", shared=65536, format="ptx",
                       image=launcher_ptx)
    tags = [abi.memref_tag(abi.F32, 1)] * 2
    abi.dispatch(blob, [abi.descriptor(ta.ptr, (16384,)),
                        abi.descriptor(ty.ptr, (16384,))], tags)
    assert np.array_equal(ty.to_host(), a[::-1])
    ta.free()
    ty.free()


ASSERT_CHILD = r"""
import ctypes as C, sys
import numpy as np
sys.path.insert(0, %(root)r)
from vx_b200 import abi
x = np.ones(256, np.float32)
x[77] = %(value)s
t = abi.DeviceTensor.from_host(x)
blob = abi.payload("vx_assert_kernel", abi=1, topo=abi.gpu(0), grid="2",
                   block="128", assert_flag=1, format="ptx",
                   image=open(%(ptx)r).read())
abi.dispatch(blob, [abi.descriptor(t.ptr, (256,))], [abi.memref_tag(abi.F32, 1)])
abi.dispatch(blob, [abi.descriptor(t.ptr, (256,))], [abi.memref_tag(abi.F32, 1)])
print("survived")
"""


def test_the_assert_flag_stops_the_program(launcher_ptx, tmp_path):
    """`assert_flag=1`: the kernel takes one more parameter, a device integer
    that a failed assert sets while the kernel runs on; the library clears it
    before and reads it after the launch (runtime/vx_kernel_launch.h:379-393).
    The failing case ends with the library's FATAL line; no GPU trap is
    involved, so it runs as an ordinary child process."""
    import sys
    ptx = tmp_path / "k.ptx"
    ptx.write_text(launcher_ptx)
    for value, ok in (("2.0", True), ("-1.0", False)):
        code = ASSERT_CHILD % dict(root=ROOT, value=value, ptx=str(ptx))
        r = subprocess.run([sys.executable, "-c", code], capture_output=True,
                           text=True, timeout=300)
        if ok:
            assert r.returncode == 0 and "survived" in r.stdout, r.stderr[-2000:]
        else:
            assert r.returncode != 0 and "survived" not in r.stdout
            assert "[Vx CUDA] FATAL: an assert failed in vx_assert_kernel" in r.stderr


def test_an_image_launch_inside_a_recording(launcher_ptx):
    """After one plain call (which loads the image) the same launch records
    into a CUDA graph on the caller's stream and replays
    (runtime/cuda_dispatch.cpp:214-244)."""
    import torch
    n = 4 * 32
    out = abi.DeviceTensor.from_host(np.zeros(n, np.int32))
    blob = abi.payload("vx_shape_kernel", abi=1, topo=abi.gpu(0), grid="4,1",
                       block="32", format="ptx", image=launcher_ptx)
    desc, tags = abi.descriptor(out.ptr, (n,)), [abi.memref_tag(abi.I32, 1),
                                                 abi.I32_KIND]
    stream = torch.cuda.Stream()
    L = lib()
    L.vx_cuda_set_stream(C.c_void_p(stream.cuda_stream))
    try:
        abi.dispatch(blob, [desc, C.c_int32(1)], tags)        # loads the image
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        value = C.c_int32(5)
        with torch.cuda.graph(graph, stream=stream,
                              capture_error_mode="thread_local"):
            abi.dispatch(blob, [desc, value], tags)
        stream.synchronize()
        assert (out.to_host() == 1 + 1000 + 32).all()         # not run yet
        graph.replay()
        stream.synchronize()
    finally:
        L.vx_cuda_set_stream(None)
    assert (out.to_host() == 5 + 1000 + 32).all()
    out.free()


def test_a_tma_copy_through_vx_plugin_tensor_map(launcher_ptx):
    """vx_plugin_tensor_map (runtime/cuda_dispatch.cpp:1966-2026): a tiled,
    unswizzled descriptor kept in device memory, one per distinct (descriptor,
    GPU); a kernel copies an 8 x 16 box through it with a plain
    cp.async.bulk.tensor (x a multiple of 4 floats = 16 bytes)."""
    L = lib()
    rows, cols = 64, 96
    src = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)
    t = abi.DeviceTensor.from_host(src)
    zero = [0] * 3

    def tensor_map(box_rows, box_cols):
        return L.vx_plugin_tensor_map(t.ptr, 2, 4, rows, cols, *zero, cols, 1,
                                      *zero, box_rows, box_cols, *zero)
    m = tensor_map(8, 16)
    assert m != 0
    assert tensor_map(8, 16) == m                 # the cache answers
    assert tensor_map(4, 16) not in (0, m)        # another box, another map
    # refusals: a base off 16 bytes, a box over 256, an inner stride other than 1
    assert L.vx_plugin_tensor_map(t.ptr + 4, 2, 4, rows, cols, *zero, cols, 1,
                                  *zero, 8, 16, *zero) == 0
    assert tensor_map(8, 512) == 0
    assert L.vx_plugin_tensor_map(t.ptr, 2, 4, rows, cols, *zero, cols, 2,
                                  *zero, 8, 16, *zero) == 0
    out = abi.DeviceTensor.from_host(np.zeros(8 * 16, np.float32))
    status = abi.DeviceTensor.from_host(np.zeros(1, np.int32))
    blob = abi.payload("vx_tma_kernel", abi=1, topo=abi.gpu(0), grid="1",
                       block="128", format="ptx", image=launcher_ptx)
    x, y = 20, 9
    tags = [abi.memref_tag(abi.F32, 1), abi.memref_tag(abi.I32, 1),
            abi.I64_KIND, abi.I32_KIND, abi.I32_KIND]
    abi.dispatch(blob, [abi.descriptor(out.ptr, (128,)),
                        abi.descriptor(status.ptr, (1,)), C.c_int64(m),
                        C.c_int32(x), C.c_int32(y)], tags)
    assert int(status.to_host()[0]) == 0, "the bounded wait for the copy ran out"
    assert np.array_equal(out.to_host().reshape(8, 16), src[y:y + 8, x:x + 16])
    for d in (t, out, status):
        d.free()
