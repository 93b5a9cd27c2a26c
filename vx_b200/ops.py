"""The operator surface, called the way a compiled Vx program calls it.

matmul / matmul_into go through vx_plugin_dispatch_async with the payload that
the compiler stamps on `c = a @ b` (name, abi=1, kind=matmul, roles=,
outkind=, topo=); the nn_* functions mirror stdlib/std/nn.vx one to one through
the vx_nn_* exports; flash_attention and gemm are the direct device-pointer
calls of include/vx_b200.h.
"""
import ctypes as C

import numpy as np

from . import abi
from .lib import check, lib


# ---- a @ b --------------------------------------------------------------------
def _matmul_payload(name, outkind, topo, roles="a:0,b:1,out:2"):
    return abi.payload(name, abi=1, kind="matmul", roles=roles,
                       outkind=outkind, topo=topo)


def matmul_into(c, a, b, name="vx_npu_kernel_0"):
    """spawn on(GPU) { matmul_into(&mut c, &a, &b) }: the result buffer is an
    operand, filled in place (outkind=buffer). a, b, c: DeviceTensor."""
    da = abi.descriptor(a.ptr, a.shape)
    db = abi.descriptor(b.ptr, b.shape)
    dc = abi.descriptor(c.ptr, c.shape)
    tags = [abi.memref_tag(t.elem, 2) for t in (a, b, c)]
    return abi.dispatch(_matmul_payload(name, "buffer", c.topo), [da, db, dc],
                        tags)


def matmul_host(a, b, topo=None, bf16=False, slot=True):
    """`c = a @ b` on operands in HOST memory: the library stages them, runs the
    product on the GPU, and either publishes a malloc'ed result through a slot
    (outkind=slot) or fills a host buffer. Returns a numpy array."""
    topo = abi.home_gpu() if topo is None else topo
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    elem = abi.code_of(a.dtype, bf16)
    m, n = a.shape[0], b.shape[1]
    da = abi.descriptor(a.ctypes.data, a.shape)
    db = abi.descriptor(b.ctypes.data, b.shape)
    if slot:
        result_desc = abi.descriptor(0, (0, 0))          # filled by the library
        slot_desc = abi.descriptor(C.addressof(result_desc), ())
        tags = [abi.memref_tag(elem, 2), abi.memref_tag(elem, 2),
                abi.memref_tag(elem, 2, slot=True)]
        abi.dispatch(_matmul_payload("vx_npu_kernel_0", "slot", topo),
                     [da, db, slot_desc], tags)
        ptr, rows, cols = result_desc[1], result_desc[3], result_desc[4]
        assert (rows, cols) == (m, n)
        nbytes = m * n * abi.DTYPE_BYTES[elem]
        out = np.frombuffer((C.c_char * nbytes).from_address(ptr),
                            dtype=abi.NUMPY_OF[elem]).reshape(m, n).copy()
        C.CDLL(None).free(C.c_void_p(ptr))   # the program's allocator owns it
        return out
    out = np.empty((m, n), dtype=abi.NUMPY_OF[elem])
    dc = abi.descriptor(out.ctypes.data, out.shape)
    tags = [abi.memref_tag(elem, 2)] * 3
    abi.dispatch(_matmul_payload("vx_npu_kernel_0", "buffer", topo),
                 [da, db, dc], tags)
    return out


def matmul(a, b):
    """Device-resident a @ b into a fresh device tensor."""
    c = abi.DeviceTensor.empty((a.shape[0], b.shape[1]), a.elem, a.topo)
    matmul_into(c, a, b)
    return c


def matvec_flat(w, x):
    """vx_plugin_dispatch_async_flat: xout[d] = W[d,n] . x, host or device."""
    d, n = w.shape
    out = np.empty(d, np.float32)
    lib().vx_plugin_dispatch_async_flat(
        out.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p),
        w.ctypes.data_as(C.c_void_p), n, d)
    return out


def wait(topo=None):
    t = C.c_int32(abi.home_gpu() if topo is None else topo)
    lib().vx_plugin_control(0x05, C.addressof(t))


def gemm(a, b, c, route=0, scratch=None):
    """Direct call on DeviceTensors (no payload)."""
    m, k = a.shape
    n = b.shape[1]
    check(lib().vx_b200_gemm(a.elem, route, m, n, k, a.ptr, k, b.ptr, n, c.ptr,
                             n, scratch.ptr if scratch is not None else None))


def kernel_status():
    return lib().vx_b200_kernel_status()


def flash_attention(q, k, v, out, scale, causal=True):
    B, H, S, D = q.shape
    check(lib().vx_b200_flash_attention(q.ptr, k.ptr, v.ptr, out.ptr, B, H, S,
                                        D, scale, int(causal)))


def fill_normal(t, seed, sigma):
    check(lib().vx_b200_fill_normal(t.ptr, int(t.elem == abi.BF16), t.count,
                                    seed, sigma))


def fill_uniform(t, seed, lo, hi):
    check(lib().vx_b200_fill_uniform(t.ptr, int(t.elem == abi.BF16), t.count,
                                     seed, lo, hi))


# ---- std::nn ---------------------------------------------------------------------
def _call(fn, *args):
    flat = []
    for a in args:
        flat += a.pub_fn_args() if isinstance(a, abi.DeviceTensor) else [a]
    getattr(lib(), fn)(*flat)


def nn_matvec(y, w, x, rows, cols):
    _call("vx_nn_matvec", y, w, x, C.c_int32(rows), C.c_int32(cols))


def nn_matvec_add(y, w, x, rows, cols):
    _call("vx_nn_matvec_add", y, w, x, C.c_int32(rows), C.c_int32(cols))


def nn_matvec_heads_add(y, w, x, rows, heads, head_dim):
    _call("vx_nn_matvec_heads_add", y, w, x, C.c_int32(rows), C.c_int32(heads),
          C.c_int32(head_dim))


def nn_qkv(q, k, v, w, b, x, q_heads, kv_heads, head_dim, cols):
    _call("vx_nn_qkv", q, k, v, w, b, x, C.c_int32(q_heads),
          C.c_int32(kv_heads), C.c_int32(head_dim), C.c_int32(cols))


def nn_swiglu(out, w, x, rows, cols):
    _call("vx_nn_swiglu", out, w, x, C.c_int32(rows), C.c_int32(cols))


def nn_rms_norm(y, x, w, n, eps):
    _call("vx_nn_rms_norm", y, x, w, C.c_int32(n), C.c_float(eps))


def nn_rope_and_store(q_out, k_cache, v_cache, q, k, v, cos, sin, pos, q_heads,
                      kv_heads, head_dim):
    _call("vx_nn_rope_and_store", q_out, k_cache, v_cache, q, k, v, cos, sin,
          C.c_int32(pos), C.c_int32(q_heads), C.c_int32(kv_heads),
          C.c_int32(head_dim))


def nn_attention_scratch_shape(max_seq, q_heads, kv_heads, head_dim):
    """nn_attention_scratch (stdlib/std/nn.vx:370-380)."""
    splits = max((max_seq + 63) // 64, 20)
    return (kv_heads * ((q_heads // kv_heads + 7) // 8), splits, 8, head_dim + 2)


def nn_attention(out, part, q, k_cache, v_cache, pos, q_heads, kv_heads,
                 head_dim):
    _call("vx_nn_attention", out, part, q, k_cache, v_cache, C.c_int32(pos),
          C.c_int32(q_heads), C.c_int32(kv_heads), C.c_int32(head_dim))


def nn_argmax(out, logits, n):
    _call("vx_nn_argmax", out, logits, C.c_int32(n))


def nn_embed(x, table, token, dim):
    _call("vx_nn_embed", x, table, token, C.c_int32(dim))


# ---- fp8 and Q4_0 weights (quant: "fp8" or "q4") ------------------------------------
def nn_matvec_quant(quant, y, w, scales, x, rows, cols, add=False):
    _call("vx_nn_matvec_%s%s" % (quant, "_add" if add else ""), y, w, scales, x,
          C.c_int32(rows), C.c_int32(cols))


def nn_matvec_quant_heads_add(quant, y, w, scales, x, rows, heads, head_dim):
    _call("vx_nn_matvec_%s_heads_add" % quant, y, w, scales, x, C.c_int32(rows),
          C.c_int32(heads), C.c_int32(head_dim))


def nn_qkv_quant(quant, q, k, v, w, scales, b, x, q_heads, kv_heads, head_dim,
                 cols):
    _call("vx_nn_qkv_%s" % quant, q, k, v, w, scales, b, x, C.c_int32(q_heads),
          C.c_int32(kv_heads), C.c_int32(head_dim), C.c_int32(cols))


def nn_swiglu_quant(quant, out, w, scales, x, rows, cols):
    _call("vx_nn_swiglu_%s" % quant, out, w, scales, x, C.c_int32(rows),
          C.c_int32(cols))


# ---- n positions at once ------------------------------------------------------------
def nn_matvec_rows(y, w, x, n, rows, cols):
    _call("vx_nn_matvec_rows", y, w, x, C.c_int32(n), C.c_int32(rows),
          C.c_int32(cols))


def nn_matvec_q4_rows(y, w, scales, x, n, rows, cols):
    _call("vx_nn_matvec_q4_rows", y, w, scales, x, C.c_int32(n), C.c_int32(rows),
          C.c_int32(cols))


def nn_rms_norm_rows(y, x, w, n, dim, eps):
    _call("vx_nn_rms_norm_rows", y, x, w, C.c_int32(n), C.c_int32(dim),
          C.c_float(eps))


def nn_argmax_rows(out, logits, n, count):
    _call("vx_nn_argmax_rows", out, logits, C.c_int32(n), C.c_int32(count))


def nn_embed_rows(x, table, tokens, n, dim):
    _call("vx_nn_embed_rows", x, table, tokens, C.c_int32(n), C.c_int32(dim))


# ---- a mixture-of-experts layer -----------------------------------------------------
def nn_top_k(ids, weights, logits, n, k):
    _call("vx_nn_top_k", ids, weights, logits, C.c_int32(n), C.c_int32(k))


def nn_moe_swiglu(out, w, ids, x, k, rows, cols, experts, scales=None):
    if scales is None:
        _call("vx_nn_moe_swiglu", out, w, ids, x, C.c_int32(k), C.c_int32(rows),
              C.c_int32(cols), C.c_int32(experts))
    else:
        _call("vx_nn_moe_swiglu_q4", out, w, scales, ids, x, C.c_int32(k),
              C.c_int32(rows), C.c_int32(cols), C.c_int32(experts))


def nn_moe_down_add(y, w, ids, weights, h, k, rows, cols, experts, scales=None):
    if scales is None:
        _call("vx_nn_moe_down_add", y, w, ids, weights, h, C.c_int32(k),
              C.c_int32(rows), C.c_int32(cols), C.c_int32(experts))
    else:
        _call("vx_nn_moe_down_q4_add", y, w, scales, ids, weights, h, C.c_int32(k),
              C.c_int32(rows), C.c_int32(cols), C.c_int32(experts))


# ---- the experts and the quantised projections of n positions -----------------------
def _i32(*values):
    return [C.c_int32(v) for v in values]


def nn_top_k_rows(ids, weights, logits, n, count, k):
    _call("vx_nn_top_k_rows", ids, weights, logits, *_i32(n, count, k))


def nn_matvec_q4_heads_add_rows(y, w, scales, x, n, rows, heads, head_dim):
    _call("vx_nn_matvec_q4_heads_add_rows", y, w, scales, x,
          *_i32(n, rows, heads, head_dim))


def nn_qkv_q4_rows(q, k, v, w, scales, b, x, n, q_heads, kv_heads, head_dim, cols):
    _call("vx_nn_qkv_q4_rows", q, k, v, w, scales, b, x,
          *_i32(n, q_heads, kv_heads, head_dim, cols))


def nn_moe_swiglu_q4_rows(out, w, scales, ids, x, n, k, rows, cols, experts):
    _call("vx_nn_moe_swiglu_q4_rows", out, w, scales, ids, x,
          *_i32(n, k, rows, cols, experts))


def nn_moe_down_q4_add_rows(y, w, scales, ids, weights, h, n, k, rows, cols, experts):
    _call("vx_nn_moe_down_q4_add_rows", y, w, scales, ids, weights, h,
          *_i32(n, k, rows, cols, experts))


# ---- pairs grouped by expert --------------------------------------------------------
def nn_moe_group_count(counts, ids, n, experts):
    _call("vx_nn_moe_group_count", counts, ids, *_i32(n, experts))


def nn_moe_group_offsets(base, starts, tile_expert, order, counts, n, experts, align):
    _call("vx_nn_moe_group_offsets", base, starts, tile_expert, order, counts,
          *_i32(n, experts, align))


def nn_moe_group_place(order, ids, base, n):
    _call("vx_nn_moe_group_place", order, ids, base, *_i32(n))


def nn_moe_group(order, counts, base, starts, tile_expert, ids, experts, align):
    _call("vx_nn_moe_group", order, counts, base, starts, tile_expert, ids,
          *_i32(experts, align))


def moe_swiglu_q4_grouped(out, w, scales, order, tile_expert, align, x, n, k, rows,
                          cols, experts):
    """The SwiGLU inputs of the experts of n positions, pairs grouped by
    nn_moe_group with `align` 8 or 16 (tile_expert gives the number of tiles)."""
    check(lib().vx_b200_moe_swiglu_q4_grouped(
        out.ptr, w.ptr, scales.ptr, order.ptr, tile_expert.ptr, tile_expert.count,
        align, x.ptr, n, k, rows, cols, experts))


def moe_down_q4_add_grouped(y, w, scales, order, tile_expert, align, weights, h,
                            scratch, n, k, rows, cols, experts):
    check(lib().vx_b200_moe_down_q4_add_grouped(
        y.ptr, w.ptr, scales.ptr, order.ptr, tile_expert.ptr, tile_expert.count,
        align, weights.ptr, h.ptr, scratch.ptr, n, k, rows, cols, experts))


def gemm_q4(y, w, scales, x, n, rows, cols):
    """y[n, rows] = x[n, cols] times the transpose of a Q4_0 matrix."""
    check(lib().vx_b200_gemm_q4(y.ptr, w.ptr, scales.ptr, x.ptr, n, rows, cols))


def gemm_fp8(y, w, scales, x, n, rows, cols):
    """y[n, rows] = x[n, cols] times the transpose of an fp8 matrix."""
    check(lib().vx_b200_gemm_fp8(y.ptr, w.ptr, scales.ptr, x.ptr, n, rows, cols))
