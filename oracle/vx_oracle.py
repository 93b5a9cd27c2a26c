"""ctypes face of the CPU oracle (oracle/vx_oracle.cpp). TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
legs import this module; nothing under vx_b200/ may.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(_build.build())
        _declare(_LIB)
    return _LIB


class LlamaConfig(C.Structure):
    """llama2.c header order used by tests/backend/pass/llama2.vx."""
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads",
                 "vocab_size", "seq_len")]


class NnConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden", "n_layers", "q_heads", "kv_heads",
                 "head_dim", "vocab", "max_seq")] + \
               [("eps", C.c_float), ("rope_theta", C.c_float)]


def _declare(L):
    i64, i32, f32 = C.c_int64, C.c_int32, C.c_float
    vp = C.c_void_p
    L.oracle_set_threads.argtypes = [C.c_int]
    L.oracle_get_threads.restype = C.c_int
    L.oracle_gemm_f32.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64]
    L.oracle_gemm_f32_rows.argtypes = L.oracle_gemm_f32.argtypes
    L.oracle_gemm_f64.argtypes = L.oracle_gemm_f32.argtypes
    L.oracle_gemm_bf16_rows.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64,
                                        vp, i64]
    L.oracle_gemm_bf16_entry.argtypes = [vp, i64, vp, i64, i64, i64, i64]
    L.oracle_gemm_bf16_entry.restype = f32
    L.oracle_matvec_f32.argtypes = [vp, vp, vp, C.c_int, C.c_int]
    L.oracle_f32_to_bf16.argtypes = [vp, vp, i64]
    L.oracle_bf16_to_f32.argtypes = [vp, vp, i64]
    L.oracle_random.argtypes = [C.c_uint32, i32, f32]
    L.oracle_random.restype = f32
    L.oracle_random_f32.argtypes = [vp, i64, C.c_uint32, f32]
    L.oracle_llama_weight_count.argtypes = [C.POINTER(LlamaConfig)]
    L.oracle_llama_weight_count.restype = i64
    L.oracle_llama_forward.argtypes = [C.POINTER(LlamaConfig), vp, vp, vp, i32,
                                       i32, vp]
    L.oracle_llama_generate.argtypes = [C.POINTER(LlamaConfig), vp, vp, i32, vp]
    L.oracle_argmax_f32.argtypes = [vp, i32]
    L.oracle_argmax_f32.restype = i32
    L.oracle_nn_matvec.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int]
    L.oracle_nn_qkv.argtypes = [vp] * 6 + [C.c_int] * 4
    L.oracle_nn_swiglu.argtypes = [vp, vp, vp, C.c_int, C.c_int]
    L.oracle_nn_rms_norm.argtypes = [vp, vp, vp, C.c_int, f32]
    L.oracle_nn_rope_and_store.argtypes = [vp] * 8 + [C.c_int] * 5
    L.oracle_nn_attention.argtypes = [vp] * 4 + [C.c_int] * 4
    L.oracle_attention_f64.argtypes = [vp] * 4 + [C.c_int] * 4
    L.oracle_nn_argmax.argtypes = [vp, i32]
    L.oracle_nn_argmax.restype = i32
    L.oracle_nn_embed.argtypes = [vp, vp, i32, C.c_int]
    L.oracle_rope_tables.argtypes = [vp, vp, C.c_int, C.c_int, C.c_double]
    L.oracle_nn_layer_params.argtypes = [C.POINTER(NnConfig)]
    L.oracle_nn_layer_params.restype = i64
    L.oracle_nn_decode_step.argtypes = [C.POINTER(NnConfig)] + [vp] * 8 + \
                                       [i32, i32, vp]
    L.oracle_nn_decode_step.restype = i32
    L.oracle_attention_rows.argtypes = [vp, vp, vp, C.c_int, C.c_int, f32,
                                        C.c_int, vp, C.c_int, vp]
    L.oracle_all_reduce_sum_f32.argtypes = [vp, C.c_int, vp, i64]
    L.oracle_nn_matvec_fp8.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int,
                                       C.c_int]
    L.oracle_nn_swiglu_fp8.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int]
    L.oracle_fp8_dot_f64.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int]
    L.oracle_nn_matvec_q4.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int]
    L.oracle_nn_swiglu_q4.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int]
    L.oracle_q4_dot_f64.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int]
    L.oracle_random_words.argtypes = [vp, i64, C.c_uint32, C.c_int]
    L.oracle_nn_top_k.argtypes = [vp, vp, vp, C.c_int, C.c_int]
    L.oracle_nn_decode_step_quant.argtypes = [C.POINTER(NnConfig), C.c_int, vp,
                                              vp, vp, vp, vp, vp, vp, vp, i32,
                                              i32, vp]
    L.oracle_nn_decode_step_quant.restype = i32


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def set_threads(n):
    lib().oracle_set_threads(int(n))


# ---- conversions -----------------------------------------------------------
def f32_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_bf16_to_f32(_p(x), _p(out), x.size)
    return out


def random_f32(n, seed, scale):
    out = np.empty(int(n), dtype=np.float32)
    lib().oracle_random_f32(_p(out), out.size, seed, scale)
    return out


# ---- GEMM --------------------------------------------------------------------
def gemm(a, b, fast=False):
    """Row-major C = A @ B for float32 or float64 arrays (k ascending)."""
    assert a.dtype == b.dtype and a.shape[1] == b.shape[0]
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), dtype=a.dtype)
    if a.dtype == np.float32:
        fn = lib().oracle_gemm_f32_rows if fast else lib().oracle_gemm_f32
    else:
        fn = lib().oracle_gemm_f64
    fn(_p(a), k, _p(b), n, _p(c), n, m, n, k)
    return c


def gemm_bf16_rows(a16, b16, rows):
    """Rows `rows` of bf16(A @ B) with an f32 accumulator; uint16 in and out."""
    a16 = np.ascontiguousarray(a16, dtype=np.uint16)
    b16 = np.ascontiguousarray(b16, dtype=np.uint16)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    k = a16.shape[1]
    n = b16.shape[1]
    c = np.empty((rows.size, n), dtype=np.uint16)
    lib().oracle_gemm_bf16_rows(_p(a16), k, _p(b16), n, _p(c), n, n, k,
                                _p(rows), rows.size)
    return c


def gemm_bf16_entry(a16, b16, i, j):
    k = a16.shape[1]
    return lib().oracle_gemm_bf16_entry(_p(a16), k, _p(b16), b16.shape[1],
                                        int(i), int(j), k)


def matvec_f32(w, x):
    d, n = w.shape
    out = np.empty(d, dtype=np.float32)
    lib().oracle_matvec_f32(_p(out), _p(np.ascontiguousarray(x)),
                            _p(np.ascontiguousarray(w)), n, d)
    return out


# ---- llama2.vx-style f32 decode ------------------------------------------------
def llama_weight_count(cfg):
    return lib().oracle_llama_weight_count(C.byref(cfg))


def llama_generate(cfg, weights, first_token, steps, want_gaps=False):
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    assert weights.size == llama_weight_count(cfg)
    tokens = np.zeros(steps + 1, dtype=np.int32)
    tokens[0] = first_token
    gaps = np.zeros(steps, dtype=np.float32)
    lib().oracle_llama_generate(C.byref(cfg), _p(weights), _p(tokens), steps,
                                _p(gaps))
    return (tokens, gaps) if want_gaps else tokens


def llama_forward(cfg, weights, kc, vc, token, pos):
    logits = np.empty(cfg.vocab_size, dtype=np.float32)
    lib().oracle_llama_forward(C.byref(cfg), _p(weights), _p(kc), _p(vc),
                               int(token), int(pos), _p(logits))
    return logits


def llama_twin_generate(cfg, weights, first_token, steps):
    """The same greedy decode by the second restatement (llama_twin.c, after
    benchmarks/llama2_100.vx with its online softmax), one thread."""
    twin = C.CDLL(_build.build_twin())
    twin.twin_generate.argtypes = [C.POINTER(LlamaConfig), C.c_void_p,
                                   C.c_void_p, C.c_int32]
    twin.twin_generate.restype = C.c_int
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    assert weights.size == llama_weight_count(cfg)
    tokens = np.zeros(steps + 1, dtype=np.int32)
    tokens[0] = first_token
    rc = twin.twin_generate(C.byref(cfg), _p(weights), _p(tokens), steps)
    assert rc == 0, "the twin needs n_kv_heads == n_heads (and memory)"
    return tokens


# ---- std::nn operators -----------------------------------------------------------
def nn_matvec(w16, x, rows, cols, y=None):
    add = y is not None
    out = np.array(y, dtype=np.float32) if add else np.empty(rows, np.float32)
    lib().oracle_nn_matvec(_p(out), _p(w16), _p(np.ascontiguousarray(x, np.float32)),
                           rows, cols, int(add))
    return out


def nn_qkv(w16, b16, x, q_heads, kv_heads, head_dim, cols):
    q = np.empty((q_heads, head_dim), np.float32)
    k = np.empty((kv_heads, head_dim), np.float32)
    v = np.empty((kv_heads, head_dim), np.float32)
    lib().oracle_nn_qkv(_p(q), _p(k), _p(v), _p(w16), _p(b16),
                        _p(np.ascontiguousarray(x, np.float32)), q_heads,
                        kv_heads, head_dim, cols)
    return q, k, v


def nn_swiglu(w16, x, rows, cols):
    out = np.empty(rows, np.float32)
    lib().oracle_nn_swiglu(_p(out), _p(w16),
                           _p(np.ascontiguousarray(x, np.float32)), rows, cols)
    return out


def nn_rms_norm(x, w16, n, eps):
    y = np.empty(n, np.float32)
    lib().oracle_nn_rms_norm(_p(y), _p(np.ascontiguousarray(x, np.float32)),
                             _p(w16), n, eps)
    return y


def rope_tables(max_seq, head_dim, theta):
    cos = np.empty((max_seq, head_dim // 2), np.float32)
    sin = np.empty_like(cos)
    lib().oracle_rope_tables(_p(cos), _p(sin), max_seq, head_dim, float(theta))
    return cos, sin


def nn_rope_and_store(k_cache, v_cache, q, k, v, cos, sin, pos):
    q_heads, head_dim = q.shape
    kv_heads = k.shape[0]
    q_out = np.empty_like(q)
    lib().oracle_nn_rope_and_store(_p(q_out), _p(k_cache), _p(v_cache), _p(q),
                                   _p(k), _p(v), _p(cos), _p(sin),
                                   cos.shape[1], pos, q_heads, kv_heads,
                                   head_dim)
    return q_out


def nn_attention(q, k_cache, v_cache, pos):
    q_heads, head_dim = q.shape
    kv_heads = k_cache.shape[1]
    out = np.empty_like(q)
    lib().oracle_nn_attention(_p(out), _p(q), _p(k_cache), _p(v_cache), pos,
                              q_heads, kv_heads, head_dim)
    return out


def attention_f64(q, k_cache, v_cache, pos):
    q_heads, head_dim = q.shape
    kv_heads = k_cache.shape[1]
    out = np.empty(q.shape, np.float64)
    lib().oracle_attention_f64(_p(out), _p(q), _p(k_cache), _p(v_cache), pos,
                               q_heads, kv_heads, head_dim)
    return out


def nn_argmax(logits):
    logits = np.ascontiguousarray(logits, np.float32)
    return lib().oracle_nn_argmax(_p(logits), logits.size)


def nn_embed(table16, token, dim):
    x = np.empty(dim, np.float32)
    lib().oracle_nn_embed(_p(x), _p(table16), int(token), dim)
    return x


def nn_layer_params(cfg):
    return lib().oracle_nn_layer_params(C.byref(cfg))


def nn_decode_step(cfg, embed, layers, final_norm, lm_head, cos, sin, kc, vc,
                   token, pos, want_logits=False):
    logits = np.empty(cfg.vocab, np.float32) if want_logits else None
    tok = lib().oracle_nn_decode_step(
        C.byref(cfg), _p(embed), _p(layers), _p(final_norm), _p(lm_head),
        _p(cos), _p(sin), _p(kc), _p(vc), int(token), int(pos),
        _p(logits) if want_logits else None)
    return (tok, logits) if want_logits else tok


# ---- fp8 and Q4_0 weights -------------------------------------------------------------
def random_words(n, seed, fp8=False):
    """u32 words of the reference tests' generator; fp8: no NaN codes."""
    out = np.empty(int(n), np.uint32)
    lib().oracle_random_words(_p(out), out.size, seed, int(fp8))
    return out


def quant_matvec(quant, w, scales, x, rows, cols, y=None, row_base=0):
    """nn_matvec_fp8 / nn_matvec_q4 (and their _add forms with y given)."""
    add = y is not None
    out = np.array(y, dtype=np.float32) if add else np.empty(rows, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    if quant == "fp8":
        lib().oracle_nn_matvec_fp8(_p(out), _p(w), _p(scales), _p(x), rows, cols,
                                   int(add), row_base)
    else:
        w = w[row_base * (cols // 8):]
        scales = scales[row_base * (cols // 32):]
        lib().oracle_nn_matvec_q4(_p(out), _p(np.ascontiguousarray(w)),
                                  _p(np.ascontiguousarray(scales)), _p(x), rows,
                                  cols, int(add))
    return out


def quant_swiglu(quant, w, scales, x, rows, cols):
    out = np.empty(rows, np.float32)
    fn = lib().oracle_nn_swiglu_fp8 if quant == "fp8" else lib().oracle_nn_swiglu_q4
    fn(_p(out), _p(w), _p(scales), _p(np.ascontiguousarray(x, np.float32)), rows,
       cols)
    return out


def quant_dot_f64(quant, w, scales, x, rows, cols):
    """Every row times x in f64 from the definition of the format."""
    want = np.empty(rows, np.float64)
    fn = lib().oracle_fp8_dot_f64 if quant == "fp8" else lib().oracle_q4_dot_f64
    fn(_p(want), _p(w), _p(scales), _p(np.ascontiguousarray(x, np.float32)), rows,
       cols)
    return want


def quant_inputs(quant, rows, cols, seed):
    """Codes and scales of a rows x cols matrix as the reference's tests make
    them: fp8 scales 0.002 + 0.001 * random (f32, one per 128 x 128 block),
    Q4_0 scales 0.003 + random * 0.001 rounded to f16 (one per 32 weights)."""
    if quant == "fp8":
        w = random_words(rows * cols // 4, seed, fp8=True)
        n = ((rows + 127) // 128) * (cols // 128)
        s = (np.float32(0.002) + np.float32(0.001) * random_f32(n, seed + 1, 1.0)) \
            .astype(np.float32)
    else:
        w = random_words(rows * (cols // 8), seed)
        n = rows * (cols // 32)
        s = (np.float32(0.003) + random_f32(n, seed + 1, 0.001)).astype(np.float16)
    return w, s


def nn_top_k(logits, k):
    """nn_top_k: (ids, weights) of the k largest of `logits` (at most 256)."""
    logits = np.ascontiguousarray(logits, np.float32)
    ids = np.empty(k, np.int32)
    weights = np.empty(k, np.float32)
    lib().oracle_nn_top_k(_p(ids), _p(weights), _p(logits), logits.size, k)
    return ids, weights


def quant_model_from_tensors(tensors, cfgd, max_seq, quant):
    """The oracle's view of a model that vx_b200.llama.nn_quant_model built on
    the GPU: per layer the 11 arrays oracle_nn_decode_step_quant reads."""
    import torch

    def host(t, dtype):
        return np.ascontiguousarray(t.cpu().numpy()).view(dtype).reshape(-1)

    L = cfgd["n_layers"]
    qkv_rows = (cfgd["q_heads"] + 2 * cfgd["kv_heads"]) * cfgd["head_dim"]
    scale_t = np.float32 if quant == "fp8" else np.uint16
    arrays = []
    for l in range(L):
        arrays += [host(tensors["attn_norm"][l].view(torch.int16), np.uint16),
                   host(tensors["wq"][l], np.uint32),
                   host(tensors["s_qkv"][l].view(torch.int16)
                        if quant == "q4" else tensors["s_qkv"][l], scale_t),
                   np.zeros(qkv_rows, np.uint16),
                   host(tensors["wo"][l], np.uint32),
                   host(tensors["s_o"][l].view(torch.int16)
                        if quant == "q4" else tensors["s_o"][l], scale_t),
                   host(tensors["ffn_norm"][l].view(torch.int16), np.uint16),
                   host(tensors["w_gate"][l], np.uint32),
                   host(tensors["s_gate_up"][l].view(torch.int16)
                        if quant == "q4" else tensors["s_gate_up"][l], scale_t),
                   host(tensors["w_down"][l], np.uint32),
                   host(tensors["s_down"][l].view(torch.int16)
                        if quant == "q4" else tensors["s_down"][l], scale_t)]
    cfg = NnConfig(cfgd["dim"], cfgd["hidden"], L, cfgd["q_heads"],
                   cfgd["kv_heads"], cfgd["head_dim"], cfgd["vocab"], max_seq,
                   1e-5, 10000.0)

    def u16(t):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)

    return dict(cfg=cfg, quant=2 if quant == "fp8" else 3, arrays=arrays,
                embed=u16(tensors["embed"]), final_norm=u16(tensors["final_norm"]),
                lm_head=u16(tensors["lm_head"]), cos=tensors["cos"],
                sin=tensors["sin"])


def quant_generate(hm, prompt, steps, max_seq):
    """nn_generate for a quantised model."""
    cfg = hm["cfg"]
    shape = (cfg.n_layers, max_seq, cfg.kv_heads, cfg.head_dim)
    kc, vc = np.zeros(shape, np.float32), np.zeros(shape, np.float32)
    ptrs = (C.c_void_p * len(hm["arrays"]))(*[a.ctypes.data for a in hm["arrays"]])
    out, pos, tok = [], 0, None

    def step(t):
        return lib().oracle_nn_decode_step_quant(
            C.byref(cfg), hm["quant"], _p(hm["embed"]), ptrs, _p(hm["final_norm"]),
            _p(hm["lm_head"]), _p(hm["cos"]), _p(hm["sin"]), _p(kc), _p(vc),
            int(t), int(pos), None)

    for t in prompt:
        tok = step(t)
        pos += 1
    for _ in range(steps):
        out.append(tok)
        tok = step(tok)
        pos += 1
    return out


# ---- a whole std::nn model on the host ------------------------------------------
def nn_model_from_tensors(tensors, cfgd, max_seq):
    """The oracle's view of a model that vx_b200.llama.nn_bf16_model built on
    the GPU (whole-model tensors: tp_ranks == 1): the per-layer weights in one
    array, in the order nn_decode_step reads them."""
    import torch

    def u16(t):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)

    L = cfgd["n_layers"]
    qkv_rows = (cfgd["q_heads"] + 2 * cfgd["kv_heads"]) * cfgd["head_dim"]
    cfg = NnConfig(cfgd["dim"], cfgd["hidden"], L, cfgd["q_heads"],
                   cfgd["kv_heads"], cfgd["head_dim"], cfgd["vocab"], max_seq,
                   1e-5, 10000.0)
    per_layer = nn_layer_params(cfg)
    flat = np.empty(L * per_layer, np.uint16)   # filled in place: 13 GB at 7B
    at = 0
    for l in range(L):
        for part in (tensors["attn_norm"][l], tensors["wq"][l], None,
                     tensors["wo"][l], tensors["ffn_norm"][l],
                     tensors["w_gate"][l], tensors["w_down"][l]):
            if part is None:                    # the q/k/v bias: zero
                flat[at:at + qkv_rows] = 0
                at += qkv_rows
            else:
                n = part.numel()
                flat[at:at + n] = u16(part).reshape(-1)
                at += n
    assert at == flat.size
    return dict(cfg=cfg, layers=flat, embed=u16(tensors["embed"]),
                final_norm=u16(tensors["final_norm"]),
                lm_head=u16(tensors["lm_head"]), cos=tensors["cos"],
                sin=tensors["sin"])


def nn_generate(hm, prompt, steps, max_seq, want_gaps=False, kv=None):
    """Feed `prompt` one token per step, then `steps` greedy steps; returns the
    generated tokens (the first is the argmax after the last prompt token),
    with want_gaps also the top-2 logit gap behind each choice. kv: caches
    [n_layers, max_seq, kv_heads, head_dim] to use instead of fresh ones."""
    cfg = hm["cfg"]
    shape = (cfg.n_layers, max_seq, cfg.kv_heads, cfg.head_dim)
    kc, vc = kv if kv is not None else (np.zeros(shape, np.float32),
                                        np.zeros(shape, np.float32))
    out, gaps, pos, tok = [], [], 0, None

    def step(t):
        if not want_gaps:
            return nn_decode_step(cfg, hm["embed"], hm["layers"],
                                  hm["final_norm"], hm["lm_head"], hm["cos"],
                                  hm["sin"], kc, vc, t, pos), 0.0
        tok, logits = nn_decode_step(
            cfg, hm["embed"], hm["layers"], hm["final_norm"], hm["lm_head"],
            hm["cos"], hm["sin"], kc, vc, t, pos, want_logits=True)
        top2 = np.partition(logits, -2)[-2:]
        return tok, float(top2[1] - top2[0])

    gap = 0.0
    for t in prompt:
        tok, gap = step(t)
        pos += 1
    for _ in range(steps):
        out.append(tok)
        gaps.append(gap)        # the gap of the step that chose this token
        tok, gap = step(tok)
        pos += 1
    return (out, gaps) if want_gaps else out


# ---- attention over sequences -------------------------------------------------------
def attention_rows(q16, k16, v16, scale, causal, rows):
    """q16,k16,v16: [S, D] uint16 (bf16) of one (batch, head)."""
    S, D = q16.shape
    rows = np.ascontiguousarray(rows, np.int32)
    out = np.empty((rows.size, D), np.float32)
    lib().oracle_attention_rows(_p(np.ascontiguousarray(q16)),
                                _p(np.ascontiguousarray(k16)),
                                _p(np.ascontiguousarray(v16)), S, D, scale,
                                int(causal), _p(rows), rows.size, _p(out))
    return out


def all_reduce_sum_f32(inputs):
    inputs = [np.ascontiguousarray(a, np.float32) for a in inputs]
    ptrs = (C.c_void_p * len(inputs))(*[a.ctypes.data for a in inputs])
    out = np.empty_like(inputs[0])
    lib().oracle_all_reduce_sum_f32(ptrs, len(inputs), _p(out), out.size)
    return out


# ---- the pairs of a mixture-of-experts layer grouped by expert ----------------------
def moe_group(ids, experts, align, room=None):
    """nn_moe_group (stdlib/std/nn.vx:1056-1294) as the plain loops its own test
    compares the kernels with (tests/optimizations/pass/
    std_nn_moe_group_sorts_pairs_by_expert.vx:83-110): a stable sort of the pairs
    by expert, each group padded to a multiple of `align`, n + i at a position i
    with no pair, -1 for a tile past the last group. counts and base follow the
    kernels' doc comments (nn.vx:1068-1069, 1105-1107): the pairs of each expert
    in each block of 256, and where the first of them goes."""
    ids = np.ascontiguousarray(ids, np.int32)
    n = ids.size
    if room is None:
        room = n + experts * (align - 1)
    tiles = (room + align - 1) // align
    order = (n + np.arange(room)).astype(np.int32)
    tile_expert = np.full(tiles, -1, np.int32)
    starts = np.zeros(experts + 1, np.int32)
    blocks = (n + 255) // 256
    counts = np.zeros((blocks, experts), np.int32)
    base = np.zeros((blocks, experts), np.int32)
    for b in range(blocks):
        counts[b] = np.bincount(ids[b * 256:(b + 1) * 256], minlength=experts)
    nxt = 0
    for e in range(experts):
        starts[e] = nxt
        members = np.flatnonzero(ids == e)
        order[nxt:nxt + members.size] = members
        padded = (members.size + align - 1) // align * align
        tile_expert[nxt // align:(nxt + padded) // align] = e
        base[:, e] = nxt + np.concatenate(([0], np.cumsum(counts[:-1, e]))) \
            if blocks else base[:, e]
        nxt += padded
    starts[experts] = nxt
    return dict(order=order, starts=starts, tile_expert=tile_expert, counts=counts,
                base=base)


def moe_group_as_the_kernels(ids, experts, align, room=None):
    """The same result by the route of the reference's three kernels: the
    per-block counts (nn.vx:1070-1102), the starts as a scan in groups of 32
    experts with a binary search for the expert of a tile (:1110-1246), and each
    pair placed after the equal ids before it in its block (:1252-1281). A second
    statement of the contract, for checking the first."""
    ids = np.ascontiguousarray(ids, np.int32)
    n = ids.size
    if room is None:
        room = n + experts * (align - 1)
    tiles = (room + align - 1) // align
    blocks = (n + 255) // 256
    counts = np.zeros((blocks, experts), np.int32)
    for b in range(blocks):
        keys = ids[b * 256:(b + 1) * 256]
        for e in range(experts):
            counts[b, e] = int(np.count_nonzero(keys == e))
    size = counts.sum(axis=0).astype(np.int64) if blocks else np.zeros(experts, np.int64)
    first = (size + align - 1) // align * align
    group = np.zeros(32, np.int64)
    for g in range(32):
        total = 0
        for x in range(32 * g, min(32 * g + 32, experts)):
            padded = first[x]
            first[x] = total
            total += padded
        group[g] = total
    before = 0
    for g in range(32):
        added = group[g]
        group[g] = before
        before += added
    end = before
    starts = np.zeros(experts + 1, np.int32)
    base = np.zeros((blocks, experts), np.int32)
    for e in range(experts):
        first[e] += group[e // 32]
        starts[e] = first[e]
        at = first[e]
        for b in range(blocks):
            base[b, e] = at
            at += counts[b, e]
    starts[experts] = end
    order = np.full(room, -7, np.int32)
    tile_expert = np.zeros(tiles, np.int32)
    for t in range(tiles):
        at = t * align
        if at < end:
            e, above = 0, experts
            while above - e > 1:
                mid = (e + above) // 2
                if first[mid] <= at:
                    e = mid
                else:
                    above = mid
            tile_expert[t] = e
            for i in range(max(first[e] + size[e], at), at + align):
                order[i] = n + i
        else:
            tile_expert[t] = -1
            for i in range(at, min(at + align, room)):
                order[i] = n + i
    for b in range(blocks):
        keys = ids[b * 256:(b + 1) * 256]
        for l in range(keys.size):
            rank = int(np.count_nonzero(keys[:l] == keys[l]))
            order[base[b, keys[l]] + rank] = b * 256 + l
    return dict(order=order, starts=starts, tile_expert=tile_expert, counts=counts,
                base=base)


def moe_group_reference_cases():
    """The six cases of the reference's test of nn_moe_group
    (std_nn_moe_group_sorts_pairs_by_expert.vx:160-203): (name, ids, experts,
    align)."""
    a = (np.arange(600) * 7 % 5).astype(np.int32)
    b = np.empty(1000, np.int32)
    state = 12345
    for p in range(1000):
        state = (state * 1103515245 + 12345) % 2147483648
        b[p] = (state // 65536) % 128
        if b[p] == 64:
            b[p] = 65
    c = np.zeros(300, np.int32)
    p = np.arange(2600)
    d = np.where(p % 2 == 1, (p // 2) % 40, 3).astype(np.int32)
    return [("600 pairs, 5 experts", a, 5, 1),
            ("1000 pairs, 160 experts", b, 160, 1),
            ("1000 pairs, 160 experts, align 16", b, 160, 16),
            ("300 pairs, 1 expert", c, 1, 1),
            ("2600 pairs, 40 experts, skewed", d, 40, 1),
            ("2600 pairs, 40 experts, skewed, align 2", d, 40, 2)]
