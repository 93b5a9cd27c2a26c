"""The producer side of the dispatch ABI, as the Vx compiler writes it: argument
tags, memref descriptors, payload blobs and topology ids
(include/vx_hardware_runtime.h), plus a device tensor that lives in memory
from vx_plugin_alloc_and_transfer.
"""
import ctypes as C

import numpy as np

from .lib import lib

# element type codes (VX_DTYPE_*)
I1, I8, I16, I32, I64, F32, F64, F16, BF16 = range(1, 10)
DTYPE_BYTES = {I1: 1, I8: 1, I16: 2, I32: 4, I64: 8, F32: 4, F64: 8, F16: 2,
               BF16: 2}
NUMPY_OF = {F32: np.float32, F64: np.float64, F16: np.float16, BF16: np.uint16,
            I32: np.int32, I64: np.int64}
I32_KIND, I64_KIND, F32_KIND = 4, 5, 6   # scalar argument kinds (VX_ABI_KIND_*)
TOPO_CPU = 0
TOPO_GPU_BASE = 500
SLOT_BIT = 1 << 24


def gpu(i=0):
    """Topology::GPU[i] as a dispatch id."""
    return TOPO_GPU_BASE + i


_home_gpu = 0


def set_home_gpu(i):
    """The GPU that tensors made without an explicit topology go to. A job
    with one process per GPU sets it to the process's own GPU (its local
    rank); GPU[0] otherwise."""
    global _home_gpu
    _home_gpu = int(i)


def home_gpu():
    return gpu(_home_gpu)


def memref_tag(elem, rank, slot=False):
    return (rank << 16) | (elem << 8) | (SLOT_BIT if slot else 0)


def code_of(dtype, bf16=False):
    if bf16:
        return BF16
    if np.dtype(dtype) == np.dtype(np.uint32):   # words of packed codes: u32 is
        return I32                               # a 32-bit integer on the wire
    for code, np_t in NUMPY_OF.items():
        if code != BF16 and np.dtype(dtype) == np.dtype(np_t):
            return code
    raise TypeError("no Vx element type for %r" % (dtype,))


def descriptor(ptr, shape, strides=None, offset=0):
    """{allocated, aligned, offset, sizes[r], strides[r]} as a ctypes array of
    int64; strides in elements, row-major when not given."""
    rank = len(shape)
    if strides is None:
        strides, step = [0] * rank, 1
        for d in range(rank - 1, -1, -1):
            strides[d] = step
            step *= shape[d]
    fields = [ptr or 0, ptr or 0, offset] + list(shape) + list(strides)
    return (C.c_int64 * len(fields))(*fields)


def payload(name, **entries):
    """name NUL key=value NUL ... in the order given."""
    blob = name.encode() + b"\0"
    for key, value in entries.items():
        blob += ("%s=%s" % (key, value)).encode() + b"\0"
    return blob


class DeviceTensor:
    """A tensor placed with transfer(x, Memory::GPU_HBM): bytes owned by the
    program until vx_plugin_free with the same topology."""

    def __init__(self, ptr, shape, elem, topo):
        self.ptr, self.shape, self.elem, self.topo = ptr, tuple(shape), elem, topo

    @property
    def count(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self):
        return self.count * DTYPE_BYTES[self.elem]

    @classmethod
    def empty(cls, shape, elem, topo=None):
        topo = home_gpu() if topo is None else topo
        n = 1
        for s in shape:
            n *= s
        ptr = lib().vx_plugin_alloc_and_transfer(
            max(n, 1) * DTYPE_BYTES[elem], None, topo, 1)
        return cls(ptr, shape, elem, topo)

    @classmethod
    def from_host(cls, array, topo=None, bf16=False, asynchronous=False):
        topo = home_gpu() if topo is None else topo
        array = np.ascontiguousarray(array)
        elem = code_of(array.dtype, bf16)
        fn = (lib().vx_plugin_alloc_and_transfer_async if asynchronous
              else lib().vx_plugin_alloc_and_transfer)
        ptr = fn(max(array.nbytes, 1), array.ctypes.data_as(C.c_void_p), topo, 1)
        return cls(ptr, array.shape, elem, topo)

    def to_host(self):
        out = np.empty(self.shape, dtype=NUMPY_OF[self.elem])
        if out.nbytes:
            lib().vx_plugin_transfer_device_to_host(
                self.ptr, out.ctypes.data_as(C.c_void_p), out.nbytes, self.topo)
        return out

    def view(self, offset_elems, shape):
        """A tensor over part of this one's memory (not owned)."""
        t = DeviceTensor(self.ptr + offset_elems * DTYPE_BYTES[self.elem],
                         shape, self.elem, self.topo)
        t._borrowed = True
        return t

    def free(self):
        if self.ptr and not getattr(self, "_borrowed", False):
            lib().vx_plugin_free(self.ptr, self.topo)
        self.ptr = None

    def pub_fn_args(self):
        """The 3 + 2r values a `pub fn` takes for this tensor."""
        d = descriptor(self.ptr, self.shape)
        vals = list(d)
        return [C.c_void_p(vals[0]), C.c_void_p(vals[1])] + \
               [C.c_int64(v) for v in vals[2:]]


def dispatch(blob, args, tags, launch_values=()):
    """vx_plugin_dispatch_async(payload, size, device_args, arg_tags, n).
    args: ctypes objects; for a memref, the descriptor array. Memref arguments
    are passed as pointer-to-pointer-to-descriptor, scalars as pointer-to-value,
    as LaunchOpLowering builds them. launch_values: the i32 values that `$j`
    in `grid=`, `block=` and `launch=` names; they sit after the n kernel
    arguments and are not counted in n."""
    n = len(args)
    extra = [C.c_int32(int(v)) for v in launch_values]
    args = list(args) + extra
    tags = list(tags) + [I32_KIND] * len(extra)
    holders, slots = [], (C.c_void_p * len(args))()
    for i, (a, tag) in enumerate(zip(args, tags)):
        if (tag & 0xFF) == 0:
            p = C.c_void_p(C.addressof(a))
            holders.append(p)
            slots[i] = C.addressof(p)
        else:
            slots[i] = C.addressof(a)
    tag_arr = (C.c_int32 * len(args))(*tags)
    buf = C.create_string_buffer(blob, len(blob))
    rc = lib().vx_plugin_dispatch_async(buf, len(blob), slots, tag_arr, n)
    holders.clear()
    return rc
