"""The C-ABI library loads without a GPU and exports every symbol that the
headers under include/ declare; host-side behaviour that needs no GPU."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from vx_b200 import build
    return build.build()


def exported(path):
    out = subprocess.run(["nm", "-D", "--defined-only", path],
                         capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if " T " in line}


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"static inline[^;{]*\{", "", text)
    return set(re.findall(r"\b(vx_[a-z0-9_]+)\s*\(", text)) - {
        n for n in re.findall(r"static inline [^(]*\b(vx_[a-z0-9_]+)\s*\(",
                              open(os.path.join(ROOT, "include", header)).read())}


def test_the_24_reference_symbols_are_exported(built):
    # tests/integration_test/abi_of_the_dispatch_library.rs:195-231
    from vx_b200.lib import REFERENCE_SYMBOLS
    assert len(REFERENCE_SYMBOLS) == 24
    missing = set(REFERENCE_SYMBOLS) - exported(built)
    assert not missing, missing


def test_every_declared_entry_point_is_exported(built):
    have = exported(built)
    for header in ("vx_hardware_runtime.h", "vx_b200.h"):
        names = declared(header)
        assert names, header
        missing = {n for n in names if n not in have}
        assert not missing, (header, missing)


def test_ctypes_can_bind_every_symbol(built):
    from vx_b200.lib import EXTRA_SYMBOLS, REFERENCE_SYMBOLS, lib
    L = lib()
    for name in REFERENCE_SYMBOLS + EXTRA_SYMBOLS:
        assert getattr(L, name)


def run_child(code):
    return subprocess.run([sys.executable, "-c", code], capture_output=True,
                          text=True, cwd=ROOT, timeout=120)


def test_host_side_calls_without_a_gpu(built):
    """What the reference's backends answer with no device present:
    host topologies give malloc memory, the stream calls keep their value,
    the worker calls say one worker, unknown opcodes answer 0."""
    from vx_b200 import abi
    from vx_b200.lib import lib
    L = lib()
    data = np.arange(16, dtype=np.float32)
    p = L.vx_plugin_alloc_and_transfer(data.nbytes, data.ctypes.data_as(C.c_void_p),
                                       abi.TOPO_CPU, 0)
    back = np.zeros_like(data)
    assert L.vx_plugin_transfer_device_to_host(p, back.ctypes.data_as(C.c_void_p),
                                               data.nbytes, abi.TOPO_CPU) == 1
    assert np.array_equal(back, data)
    L.vx_plugin_free(p, abi.TOPO_CPU)
    assert L.vx_host_worker_id() == 0 and L.vx_host_worker_count() == 1
    assert L.vx_cuda_get_stream() is None
    L.vx_cuda_set_stream(C.c_void_p(0x1234))
    assert L.vx_cuda_get_stream() == 0x1234
    L.vx_cuda_set_stream(None)
    assert L.vx_plugin_control(0x7777, None) == 0
    pair = (C.c_int32 * 2)(3456, 501)
    assert L.vx_plugin_control(0x04, C.addressof(pair)) == 1
    assert L.vx_plugin_control(0x04, C.addressof(pair)) == 1     # same pair again
    assert L.vx_plugin_control(0x04, None) == 0


def test_collectives_in_a_job_of_one_rank():
    """tests/backend/pass/collectives_in_a_job_of_one_rank.vx:
    CHECK: -1 0, 0 1, -1 0, 1.5 2.5, 3 3, 1 2 3, 4 4 (no GPU: a job of one)."""
    code = r'''
import ctypes as C, numpy as np, torch
from vx_b200.lib import lib
L = lib()
if torch.cuda.is_available():
    raise SystemExit(0)
print(L.vx_collective_rank(), L.vx_collective_ranks())
L.vx_collective_init(0, 1)
print(L.vx_collective_rank(), L.vx_collective_ranks())
a = np.array([1.5, 2.5], np.float32); o = np.zeros(2, np.float32)
L.vx_collective_all_reduce_sum_f32(a.ctypes.data, o.ctypes.data, 2); print(o[0], o[1])
b = np.array([3, 3], np.uint16); ob = np.zeros(2, np.uint16)
L.vx_collective_all_reduce_sum_bf16(b.ctypes.data, ob.ctypes.data, 2); print(ob[0], ob[1])
g = np.array([1, 2, 3], np.float32); og = np.zeros(3, np.float32)
L.vx_collective_all_gather_f32(g.ctypes.data, og.ctypes.data, 3); print(*og.astype(int))
L.vx_collective_all_gather_bf16(b.ctypes.data, ob.ctypes.data, 2)
L.vx_collective_finish()
print(L.vx_collective_rank(), L.vx_collective_ranks())
'''
    r = run_child(code)
    assert r.returncode == 0, r.stderr
    if r.stdout.strip():
        assert r.stdout.split() == "-1 0 0 1 1.5 2.5 3 3 1 2 3 -1 0".split()


@pytest.mark.parametrize("what,code,message", [
    ("second init", "L.vx_collective_init(0, 1); L.vx_collective_init(0, 1)",
     "second time"),
    ("two ranks, no GPU", "L.vx_collective_init(0, 2)", "one rank only"),
    ("finish before init", "L.vx_collective_finish()", "before vx_collective_init"),
])
def test_collective_misuse_stops_the_program(what, code, message):
    r = run_child("import torch\nfrom vx_b200.lib import lib\nL = lib()\n"
                  "import sys\nif torch.cuda.is_available(): sys.exit(0)\n" + code)
    if r.returncode == 0:
        pytest.skip("a GPU is present: the NCCL path answers instead")
    assert r.returncode < 0 and "FATAL" in r.stderr and message in r.stderr


def test_a_gpu_region_without_a_gpu_stops_with_a_message():
    """No host fallback: a `kind=matmul` region placed on GPU[0] on a machine
    with no GPU is a FATAL, not a CPU computation."""
    code = r'''
import numpy as np, torch, sys
if torch.cuda.is_available(): sys.exit(0)
from vx_b200 import ops
ops.matmul_host(np.ones((2, 2), np.float32), np.ones((2, 2), np.float32))
print("computed")
'''
    r = run_child(code)
    if r.returncode == 0:
        pytest.skip("a GPU is present")
    assert "computed" not in r.stdout
    assert "FATAL" in r.stderr and "no host fallback" in r.stderr


def test_payload_and_descriptor_builders_match_the_wire_format():
    from vx_b200 import abi
    blob = abi.payload("vx_npu_kernel_0", abi=1, kind="matmul",
                       roles="a:0,b:1,out:2", outkind="buffer", topo=500)
    # tests/optimizations/pass/kernel_kind_matmul.vx PAYLOAD:
    assert b"\0kind=matmul\0roles=a:0,b:1,out:2\0outkind=buffer\0" in blob
    assert blob.startswith(b"vx_npu_kernel_0\0abi=1\0") and blob.endswith(b"topo=500\0")
    d = abi.descriptor(0x1000, (3, 5))
    assert list(d) == [0x1000, 0x1000, 0, 3, 5, 5, 1]
    assert abi.memref_tag(abi.BF16, 2) == (2 << 16) | (9 << 8)
    assert abi.memref_tag(abi.F32, 2, slot=True) == (1 << 24) | (2 << 16) | (6 << 8)
    assert abi.gpu(3) == 503


def test_llama2c_header_is_read_and_checked(tmp_path):
    """vx_b200_llama2c_config (the reference's vx_load_config,
    stdlib/rust_core/src/ffi/llama.rs:11-27): no GPU involved."""
    import ctypes as C
    import numpy as np
    from vx_b200 import llama
    from vx_b200.lib import Llama2cConfig, lib
    L = lib()
    shape = dict(dim=64, hidden=176, n_layers=2, n_heads=4, n_kv_heads=4,
                 vocab=512, seq_len=32)
    flat, _ = llama.small_f32_weights(**shape)
    good = tmp_path / "model.bin"
    llama.write_llama2c(str(good), flat, **shape)
    head = Llama2cConfig()
    assert L.vx_b200_llama2c_config(str(good).encode(), C.byref(head)) == 0
    assert (head.dim, head.hidden_dim, head.n_layers, head.n_heads,
            head.n_kv_heads, head.vocab_size, head.seq_len) == (64, 176, 2, 4, 4, 512, 32)
    assert L.vx_b200_llama2c_config(str(tmp_path / "none.bin").encode(), None) == -1
    assert b"cannot open" in L.vx_b200_last_error()
    short = tmp_path / "short.bin"
    short.write_bytes(good.read_bytes()[:4096])
    assert L.vx_b200_llama2c_config(str(short).encode(), None) == -1
    assert b"cut short" in L.vx_b200_last_error()
    junk = tmp_path / "junk.bin"
    junk.write_bytes(np.zeros(64, np.int32).tobytes())
    assert L.vx_b200_llama2c_config(str(junk).encode(), None) == -1
    assert b"does not begin with a llama2.c header" in L.vx_b200_last_error()


@pytest.mark.parametrize("call,message", [
    ("ops.nn_moe_group_count(t((1, 4)), t((10,)), 10, 0)",
     "nn_moe_group_count: `experts` must be 1 to 1024"),
    ("ops.nn_moe_group_count(t((1, 4)), t((600,)), 600, 4)",
     "`counts` needs a row for each 256 pairs"),
    ("ops.nn_moe_group_offsets(t((1, 4)), t((5,)), t((3,)), t((20,)), t((1, 4)), 10, 4, 8)",
     "`order` needs n + experts * (align - 1) positions"),
    ("ops.nn_moe_group_place(t((10,)), t((5,)), t((1, 4)), 10)",
     "nn_moe_group_place: `ids` needs n values"),
    ("ops.nn_top_k_rows(t((5, 4)), t((5, 4), abi.F32), t((5, 16), abi.F32), 5, 16, 17)",
     "nn_top_k_rows: count must be 1 to 256, and k must be 1 to count"),
    ("ops.nn_moe_swiglu_q4_rows(t((19, 64), abi.F32), t((100,)), t((100,), abi.F16), "
     "t((5, 4)), t((5, 256), abi.F32), 5, 4, 64, 256, 16)",
     "`out` a row of rows values for each of the n * k"),
])
def test_refused_shapes_of_the_expert_functions_stop_with_the_function_name(call, message):
    """The asserts of nn_moe_group_count / _offsets / _place, nn_top_k_rows and
    nn_moe_swiglu_q4_rows (stdlib/std/nn.vx:1071-1072, 1111-1113, 1253, 2898-2900,
    2959) are checked before anything touches the GPU: a refused shape stops
    the program with the function's name, with or without a GPU."""
    code = ("from vx_b200 import abi, ops\n"
            "def t(shape, elem=abi.I32):\n"
            "    return abi.DeviceTensor(0x10000, shape, elem, 0)\n" + call + "\n"
            "print('went on')\n")
    r = run_child(code)
    assert r.returncode < 0 and "went on" not in r.stdout, r.stderr[-500:]
    assert "FATAL" in r.stderr and message in r.stderr, r.stderr[-500:]
