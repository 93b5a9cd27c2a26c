"""Load libvx_cuda_dispatch.so and declare its C entry points.

The library is the product: if it has not been built this module raises, and
nothing in the package computes anything without it.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("VX_DISPATCH_LIB",
                          os.path.join(HERE, "libvx_cuda_dispatch.so"))

# The exports of include/vx_hardware_runtime.h plus the two stream calls and
# the two host-worker calls: what the reference's ABI test looks for
# (tests/integration_test/abi_of_the_dispatch_library.rs:195-231).
REFERENCE_SYMBOLS = [
    "vx_plugin_alloc_and_transfer", "vx_plugin_alloc_and_transfer_async",
    "vx_plugin_dispatch_async", "vx_plugin_dispatch_async_flat",
    "vx_plugin_await_future", "vx_plugin_release_future",
    "vx_plugin_transfer_device_to_host", "vx_plugin_transfer_peer",
    "vx_plugin_free", "vx_plugin_arrivals_take", "vx_plugin_arrivals_give",
    "vx_plugin_control",
    "vx_collective_init", "vx_collective_finish", "vx_collective_rank",
    "vx_collective_ranks", "vx_collective_all_reduce_sum_f32",
    "vx_collective_all_reduce_sum_bf16", "vx_collective_all_gather_f32",
    "vx_collective_all_gather_bf16",
    "vx_host_worker_id", "vx_host_worker_count",
    "vx_cuda_set_stream", "vx_cuda_get_stream",
]
EXTRA_SYMBOLS = [
    "vx_plugin_tensor_map",
    "vx_nn_matvec", "vx_nn_matvec_add", "vx_nn_matvec_heads_add", "vx_nn_qkv",
    "vx_nn_swiglu", "vx_nn_rms_norm", "vx_nn_rope_and_store",
    "vx_nn_attention", "vx_nn_argmax", "vx_nn_embed",
    "vx_nn_matvec_fp8", "vx_nn_matvec_fp8_add", "vx_nn_matvec_fp8_heads_add",
    "vx_nn_qkv_fp8", "vx_nn_swiglu_fp8",
    "vx_nn_matvec_q4", "vx_nn_matvec_q4_add", "vx_nn_matvec_q4_heads_add",
    "vx_nn_qkv_q4", "vx_nn_swiglu_q4",
    "vx_nn_matvec_rows", "vx_nn_matvec_q4_rows", "vx_nn_rms_norm_rows",
    "vx_nn_argmax_rows", "vx_nn_embed_rows",
    "vx_nn_top_k_rows", "vx_nn_matvec_q4_heads_add_rows", "vx_nn_qkv_q4_rows",
    "vx_nn_moe_swiglu_q4_rows", "vx_nn_moe_down_q4_add_rows",
    "vx_nn_moe_group_count", "vx_nn_moe_group_offsets", "vx_nn_moe_group_place",
    "vx_nn_moe_group",
    "vx_nn_top_k", "vx_nn_moe_swiglu", "vx_nn_moe_down_add", "vx_nn_moe_swiglu_q4",
    "vx_nn_moe_down_q4_add",
    "vx_decoder_create", "vx_decoder_destroy", "vx_decoder_reset",
    "vx_decoder_step", "vx_decoder_prefill", "vx_decoder_logits",
    "vx_decoder_kernels_per_step",
    "vx_decoder_step_trace",
    "vx_decoder_kv_cache", "vx_decoder_kv_cache_bytes", "vx_decoder_adopt_kv",
    "vx_decoder_stream", "vx_b200_llama2c_config", "vx_decoder_from_llama2c",
    "vx_b200_last_error", "vx_b200_gemm", "vx_b200_kernel_status",
    "vx_b200_flash_attention", "vx_b200_gemm_column_split",
    "vx_b200_fill_normal", "vx_b200_fill_uniform", "vx_b200_quantize",
    "vx_b200_attention_decode_static", "vx_b200_attention_kernel",
    "vx_b200_moe_swiglu_q4_grouped", "vx_b200_moe_down_q4_add_grouped",
    "vx_b200_gemm_q4", "vx_b200_gemm_fp8",
]

_lib = None


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden", "n_layers", "q_heads", "kv_heads",
                 "head_dim", "vocab", "max_seq")] + \
               [("eps", C.c_float), ("rope_theta", C.c_float),
                ("weights_bf16", C.c_int32), ("batch", C.c_int32),
                ("tp_ranks", C.c_int32), ("tp_reduce", C.c_int32)]


class DecoderWeights(C.Structure):
    _fields_ = [("embed", C.c_void_p)] + \
               [(n, C.POINTER(C.c_void_p)) for n in
                ("attn_norm", "wq", "wk", "wv", "bqkv", "wo", "ffn_norm",
                 "w_gate", "w_up", "w_down")] + \
               [("final_norm", C.c_void_p), ("lm_head", C.c_void_p),
                ("cos", C.c_void_p), ("sin", C.c_void_p)] + \
               [(n, C.POINTER(C.c_void_p)) for n in
                ("s_qkv", "s_o", "s_gate_up", "s_down")]


class Llama2cConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads",
                 "vocab_size", "seq_len")]


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libvx_cuda_dispatch.so is not built (%s). Run "
            "`python -m vx_b200.build`; there is no fallback." % LIB_PATH)
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, sz, u32, i32, i64, u64 = (C.c_void_p, C.c_size_t, C.c_uint32,
                                  C.c_int32, C.c_int64, C.c_uint64)
    L.vx_plugin_alloc_and_transfer.restype = vp
    L.vx_plugin_alloc_and_transfer.argtypes = [sz, vp, u32, u32]
    L.vx_plugin_alloc_and_transfer_async.restype = vp
    L.vx_plugin_alloc_and_transfer_async.argtypes = [sz, vp, u32, u32]
    L.vx_plugin_dispatch_async.restype = u64
    L.vx_plugin_dispatch_async.argtypes = [vp, sz, C.POINTER(vp),
                                           C.POINTER(i32), i64]
    L.vx_plugin_dispatch_async_flat.restype = u64
    L.vx_plugin_dispatch_async_flat.argtypes = [vp, vp, vp, C.c_int, C.c_int]
    L.vx_plugin_await_future.argtypes = [u64]
    L.vx_plugin_release_future.argtypes = [u64]
    L.vx_plugin_transfer_device_to_host.restype = i32
    L.vx_plugin_transfer_device_to_host.argtypes = [vp, vp, sz, u32]
    L.vx_plugin_transfer_peer.restype = vp
    L.vx_plugin_transfer_peer.argtypes = [vp, u32, u32, sz]
    L.vx_plugin_free.argtypes = [vp, u32]
    L.vx_plugin_arrivals_take.restype = vp
    L.vx_plugin_arrivals_take.argtypes = [vp, sz, vp, u32, u32]
    L.vx_plugin_arrivals_give.argtypes = [vp, vp, sz, u32]
    L.vx_plugin_control.restype = i32
    L.vx_plugin_control.argtypes = [u32, vp]
    L.vx_plugin_tensor_map.restype = i64
    L.vx_plugin_tensor_map.argtypes = [i64] * 18
    L.vx_collective_init.argtypes = [i32, i32]
    L.vx_collective_rank.restype = i32
    L.vx_collective_ranks.restype = i32
    for n in ("all_reduce_sum_f32", "all_reduce_sum_bf16", "all_gather_f32",
              "all_gather_bf16"):
        getattr(L, "vx_collective_" + n).argtypes = [vp, vp, i64]
    L.vx_host_worker_id.restype = i64
    L.vx_host_worker_count.restype = i64
    L.vx_cuda_set_stream.argtypes = [vp]
    L.vx_cuda_get_stream.restype = vp
    L.vx_decoder_create.restype = vp
    L.vx_decoder_create.argtypes = [C.POINTER(DecoderConfig),
                                    C.POINTER(DecoderWeights)]
    L.vx_decoder_destroy.argtypes = [vp]
    L.vx_decoder_reset.argtypes = [vp]
    L.vx_decoder_step.restype = i32
    L.vx_decoder_step.argtypes = [vp, vp, vp]
    L.vx_decoder_prefill.restype = i32
    L.vx_decoder_prefill.argtypes = [vp, vp, i32]
    L.vx_decoder_logits.restype = vp
    L.vx_decoder_logits.argtypes = [vp]
    L.vx_decoder_kv_cache.restype = vp
    L.vx_decoder_kv_cache.argtypes = [vp, i32]
    L.vx_decoder_kv_cache_bytes.restype = i64
    L.vx_decoder_kv_cache_bytes.argtypes = [vp]
    L.vx_decoder_adopt_kv.restype = i32
    L.vx_decoder_adopt_kv.argtypes = [vp, vp, vp, i32]
    L.vx_decoder_step_trace.restype = i32
    L.vx_decoder_step_trace.argtypes = [vp, vp, i32]
    L.vx_decoder_kernels_per_step.restype = i32
    L.vx_decoder_kernels_per_step.argtypes = [vp]
    L.vx_decoder_stream.restype = vp
    L.vx_decoder_stream.argtypes = [vp]
    L.vx_b200_last_error.restype = C.c_char_p
    L.vx_b200_gemm.restype = i32
    L.vx_b200_gemm.argtypes = [i32, i32, i64, i64, i64, vp, i64, vp, i64, vp,
                               i64, vp]
    L.vx_b200_kernel_status.restype = i32
    L.vx_b200_flash_attention.restype = i32
    L.vx_b200_flash_attention.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32,
                                          C.c_float, i32]
    L.vx_b200_gemm_column_split.restype = i32
    L.vx_b200_gemm_column_split.argtypes = [i32, i64, i64, i64, vp, vp, vp, vp,
                                            vp]
    L.vx_b200_fill_normal.restype = i32
    L.vx_b200_fill_normal.argtypes = [vp, i32, i64, u64, C.c_float]
    L.vx_b200_fill_uniform.restype = i32
    L.vx_b200_fill_uniform.argtypes = [vp, i32, i64, u64, C.c_float, C.c_float]
    L.vx_b200_attention_decode_static.restype = i32
    L.vx_b200_attention_decode_static.argtypes = [vp, vp, vp, vp, i32, i32, i32,
                                                  i32]
    L.vx_b200_quantize.restype = i32
    L.vx_b200_quantize.argtypes = [i32, vp, i32, i32, vp, vp]
    L.vx_b200_llama2c_config.restype = i32
    L.vx_b200_llama2c_config.argtypes = [C.c_char_p, vp]
    L.vx_decoder_from_llama2c.restype = vp
    L.vx_decoder_from_llama2c.argtypes = [C.c_char_p, i32, i32]
    L.vx_b200_attention_kernel.restype = i32
    L.vx_b200_attention_kernel.argtypes = [i32]
    L.vx_b200_gemm_fp8.restype = i32
    L.vx_b200_gemm_fp8.argtypes = [vp, vp, vp, vp, i32, i32, i32]
    L.vx_b200_gemm_q4.restype = i32
    L.vx_b200_gemm_q4.argtypes = [vp, vp, vp, vp, i32, i32, i32]
    L.vx_b200_moe_swiglu_q4_grouped.restype = i32
    L.vx_b200_moe_swiglu_q4_grouped.argtypes = [vp] * 5 + [i32, i32, vp] + [i32] * 5
    L.vx_b200_moe_down_q4_add_grouped.restype = i32
    L.vx_b200_moe_down_q4_add_grouped.argtypes = [vp] * 5 + [i32, i32, vp, vp, vp] + [i32] * 5
    _lib = L
    return L


def check(rc):
    if rc != 0:
        raise RuntimeError(lib().vx_b200_last_error().decode())
