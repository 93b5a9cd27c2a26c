"""Llama-2-architecture decoders on the whole-token entry points
(vx_decoder_*, include/vx_b200.h).

Two flavours, as the reference has them:
  * `small_f32_model`: f32 weights in llama2.c order, interleaved RoPE, shared
    classifier -- the program tests/backend/pass/llama2.vx runs;
  * `nn_bf16_model`: bf16 weights in the layouts of stdlib/std/nn.vx
    (q, k, v rows; gate then up rows), half-split RoPE from tables.
Weights are synthetic: N(0, 0.02^2) matrices and embeddings, RMSNorm gains of 1
(the usual random initialisation of this architecture).
"""
import ctypes as C

import numpy as np

from . import abi
from .lib import DecoderConfig, DecoderWeights, Llama2cConfig, lib


def _ptr_array(ptrs):
    arr = (C.c_void_p * len(ptrs))(*[p or None for p in ptrs])
    return arr


class Decoder:
    """One vx_decoder. `weights` maps field -> list of device pointers (per
    layer) or a single pointer; `keep` holds whatever owns that memory."""

    @classmethod
    def from_llama2c(cls, path, batch=1, max_seq=0):
        """A decoder over a llama2.c checkpoint file (the reference's
        vx_load_config + vx_load_weights, stdlib/rust_core/src/ffi/llama.rs):
        the library reads the file and owns the weights on the GPU."""
        L = lib()
        head = Llama2cConfig()
        if L.vx_b200_llama2c_config(path.encode(), C.byref(head)) != 0:
            raise RuntimeError(L.vx_b200_last_error().decode())
        handle = L.vx_decoder_from_llama2c(path.encode(), batch, max_seq)
        if not handle:
            raise RuntimeError(L.vx_b200_last_error().decode())
        self = cls.__new__(cls)
        self.cfg = DecoderConfig(
            dim=head.dim, hidden=head.hidden_dim, n_layers=head.n_layers,
            q_heads=head.n_heads, kv_heads=head.n_kv_heads,
            head_dim=head.dim // head.n_heads, vocab=head.vocab_size,
            max_seq=max_seq or head.seq_len, eps=1e-5, rope_theta=10000.0,
            weights_bf16=0, batch=batch, tp_ranks=1, tp_reduce=0)
        self.keep, self._arrays, self._w, self.handle = None, {}, None, handle
        self._in = (C.c_int32 * 32)()
        self._out = (C.c_int32 * 32)()
        return self

    def __init__(self, cfg, weights, keep=None):
        self.cfg = cfg
        self.keep = keep
        self._arrays = {}
        w = DecoderWeights()
        for name, value in weights.items():
            if isinstance(value, (list, tuple)):
                arr = _ptr_array(value)
                self._arrays[name] = arr
                setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
            else:
                setattr(w, name, value)
        self._w = w
        self.handle = lib().vx_decoder_create(C.byref(cfg), C.byref(w))
        self._in = (C.c_int32 * 32)()
        self._out = (C.c_int32 * 32)()

    def reset(self):
        lib().vx_decoder_reset(self.handle)

    def step(self, tokens=None, fetch=True):
        """tokens: `batch` ints, or None to feed the previous argmax. Returns
        the argmax tokens (a list) when fetch, else None."""
        tin = None
        if tokens is not None:
            for i, t in enumerate(tokens):
                self._in[i] = int(t)
            tin = C.addressof(self._in)
        lib().vx_decoder_step(self.handle, tin,
                              C.addressof(self._out) if fetch else None)
        return [self._out[i] for i in range(self.cfg.batch)] if fetch else None

    def prefill(self, tokens):
        """Feed a prompt (one sequence): all positions but the last in one pass
        where the decoder can (vx_decoder_prefill), single steps otherwise.
        Returns the argmax after the last prompt token."""
        tokens = [int(t) for t in tokens]
        head = tokens[:-1]
        taken = 0
        if head:
            arr = (C.c_int32 * len(head))(*head)
            taken = lib().vx_decoder_prefill(self.handle, arr, len(head))
            if taken < 0:
                taken = 0
        for t in head[taken:]:
            self.step([t], fetch=False)
        return self.step([tokens[-1]])[0]

    def logits(self):
        """[batch, local vocab] f32 from the last step."""
        n = self.cfg.batch * (self.cfg.vocab // max(self.cfg.tp_ranks, 1))
        out = np.empty(n, np.float32)
        lib().vx_plugin_transfer_device_to_host(
            lib().vx_decoder_logits(self.handle),
            out.ctypes.data_as(C.c_void_p), out.nbytes, abi.home_gpu())
        return out.reshape(self.cfg.batch, -1)

    @property
    def stream(self):
        return lib().vx_decoder_stream(self.handle)

    def kv_cache(self, which):
        """Device address of the K (0) or V (1) cache; kv_cache_bytes each."""
        return lib().vx_decoder_kv_cache(self.handle, which)

    @property
    def kv_cache_bytes(self):
        return lib().vx_decoder_kv_cache_bytes(self.handle)

    def adopt_kv(self, k, v, positions):
        """Take over rows 0..positions-1 of caches laid out like this decoder's
        (device addresses, any GPU of the process) and continue from there."""
        got = lib().vx_decoder_adopt_kv(self.handle, k, v, positions)
        if got < 0:
            raise ValueError(lib().vx_b200_last_error().decode())
        return got

    def step_trace(self):
        """[projections, 6] uint64 nanosecond readings of the last step (a
        decoder made with VXB_STEP_TRACE=1 whose step is one launch), else
        None."""
        if not self.handle:
            raise ValueError("the decoder is closed")
        out = np.zeros(6 * (4 * self.cfg.n_layers + 1), np.uint64)
        n = lib().vx_decoder_step_trace(self.handle,
                                        out.ctypes.data_as(C.c_void_p), out.size)
        return out[:n].reshape(-1, 6) if n else None

    @property
    def kernels_per_step(self):
        if not self.handle:
            raise ValueError("the decoder is closed")
        return lib().vx_decoder_kernels_per_step(self.handle)

    def close(self):
        if self.handle:
            lib().vx_decoder_destroy(self.handle)
            self.handle = None


def write_llama2c(path, flat, dim, hidden, n_layers, n_heads, n_kv_heads, vocab,
                  seq_len):
    """A llama2.c checkpoint with a shared classifier: the 7 int32 of the header,
    then the f32 weights in the order of small_f32_weights()."""
    with open(path, "wb") as f:
        f.write(np.array([dim, hidden, n_layers, n_heads, n_kv_heads, vocab,
                          seq_len], np.int32).tobytes())
        f.write(np.ascontiguousarray(flat, np.float32).tobytes())


# ---- the f32 program's model ---------------------------------------------------
def small_f32_weights(dim=288, hidden=768, n_layers=6, n_heads=6, n_kv_heads=6,
                      vocab=32000, seq_len=256, seed=42):
    """One flat f32 array in llama2.c order (memory_map_weights,
    tests/backend/pass/llama2.vx:125-147) and the offsets of its parts."""
    hs = dim // n_heads
    kv = n_kv_heads * hs
    sizes = [("tok", vocab * dim), ("rms_att", n_layers * dim),
             ("wq", n_layers * dim * dim), ("wk", n_layers * dim * kv),
             ("wv", n_layers * dim * kv), ("wo", n_layers * dim * dim),
             ("rms_ffn", n_layers * dim), ("w1", n_layers * dim * hidden),
             ("w2", n_layers * hidden * dim), ("w3", n_layers * dim * hidden),
             ("rms_final", dim)]
    offsets, at = {}, 0
    for name, n in sizes:
        offsets[name] = (at, n)
        at += n
    rng = np.random.default_rng(seed)
    flat = (rng.standard_normal(at, dtype=np.float32) * np.float32(0.02))
    for name in ("rms_att", "rms_ffn", "rms_final"):
        o, n = offsets[name]
        flat[o:o + n] = 1.0
    return flat, offsets


def small_f32_decoder(flat, offsets, dim=288, hidden=768, n_layers=6, n_heads=6,
                      n_kv_heads=6, vocab=32000, seq_len=256, batch=1):
    hs = dim // n_heads
    kv = n_kv_heads * hs
    dev = abi.DeviceTensor.from_host(flat)      # one transfer, then views

    def part(name, layer=None, per_layer=None):
        o, n = offsets[name]
        if layer is not None:
            o += layer * per_layer
        return dev.ptr + 4 * o

    L = range(n_layers)
    weights = dict(
        embed=part("tok"),
        attn_norm=[part("rms_att", l, dim) for l in L],
        wq=[part("wq", l, dim * dim) for l in L],
        wk=[part("wk", l, dim * kv) for l in L],
        wv=[part("wv", l, dim * kv) for l in L],
        wo=[part("wo", l, dim * dim) for l in L],
        ffn_norm=[part("rms_ffn", l, dim) for l in L],
        w_gate=[part("w1", l, dim * hidden) for l in L],
        w_up=[part("w3", l, dim * hidden) for l in L],
        w_down=[part("w2", l, hidden * dim) for l in L],
        final_norm=part("rms_final"),
        lm_head=part("tok"),
    )
    cfg = DecoderConfig(dim=dim, hidden=hidden, n_layers=n_layers,
                        q_heads=n_heads, kv_heads=n_kv_heads, head_dim=hs,
                        vocab=vocab, max_seq=seq_len, eps=1e-5,
                        rope_theta=10000.0, weights_bf16=0, batch=batch,
                        tp_ranks=1, tp_reduce=0)
    return Decoder(cfg, weights, keep=dev)


# ---- tensor-parallel slices --------------------------------------------------------
def tp_slices(q_heads, kv_heads, head_dim, hidden, vocab, rank, ranks):
    """Which part of every matrix rank `rank` of `ranks` holds. Column-split
    projections (q, k, v, gate, up, classifier) give row ranges of the stored
    [rows, cols] matrix; row-split projections (output, down) give column
    ranges, and their partial products are summed across ranks."""
    assert q_heads % ranks == 0 and kv_heads % ranks == 0
    assert hidden % ranks == 0 and vocab % ranks == 0
    ql, kvl, hl, vl = (q_heads // ranks, kv_heads // ranks, hidden // ranks,
                       vocab // ranks)
    q0 = rank * ql * head_dim
    k0 = q_heads * head_dim + rank * kvl * head_dim
    v0 = (q_heads + kv_heads) * head_dim + rank * kvl * head_dim
    return dict(
        q_rows=(q0, q0 + ql * head_dim),              # of the fused qkv matrix
        k_rows=(k0, k0 + kvl * head_dim),
        v_rows=(v0, v0 + kvl * head_dim),
        wo_cols=(rank * ql * head_dim, (rank + 1) * ql * head_dim),
        gate_rows=(rank * hl, (rank + 1) * hl),       # of the fused gate/up
        up_rows=(hidden + rank * hl, hidden + (rank + 1) * hl),
        down_cols=(rank * hl, (rank + 1) * hl),
        vocab_rows=(rank * vl, (rank + 1) * vl),
        q_local=ql, kv_local=kvl, hidden_local=hl, vocab_local=vl)


# ---- the std::nn model -------------------------------------------------------------
def rope_tables(max_seq, head_dim, theta):
    """cos/sin [max_seq, head_dim/2] as the reference's test makes them
    (std_nn_kernels_match_loops_on_the_cpu.vx:262-272): f64 angle, f32 table."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    p = np.arange(max_seq, dtype=np.float64)[:, None]
    angle = p / np.power(float(theta), 2.0 * i / head_dim)[None, :]
    return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


def nn_bf16_model(dim, hidden, n_layers, q_heads, kv_heads, head_dim, vocab,
                  max_seq, seed=7, batch=1, tp_rank=0, tp_ranks=1,
                  theta=10000.0, eps=1e-5, device=None, tp_reduce=1):
    """Build the model on the GPU (torch only holds the memory). Every value is
    a function of (seed, tensor, element index), so all tensor-parallel degrees
    see the same model; a rank keeps its slice. Returns (Decoder, tensors) where
    tensors has the WHOLE-model layer tensors only when tp_ranks == 1."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None \
        else device
    L = lib()

    def normal(shape, tensor_id):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        rc = L.vx_b200_fill_normal(t.data_ptr(), 1, t.numel(),
                                   seed * 1000003 + tensor_id, 0.02)
        assert rc == 0, L.vx_b200_last_error()
        return t

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device=dev)

    sl = tp_slices(q_heads, kv_heads, head_dim, hidden, vocab, tp_rank, tp_ranks)

    def rows(t, r):
        return t[r[0]:r[1]].clone()

    def cols(t, r):
        return t[:, r[0]:r[1]].contiguous()

    keep = {k: [] for k in ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm",
                            "w_gate", "w_up", "w_down")}
    for l in range(n_layers):
        base = 16 * (l + 1)
        wqkv = normal(((q_heads + 2 * kv_heads) * head_dim, dim), base + 0)
        wo = normal((dim, q_heads * head_dim), base + 1)
        wgu = normal((2 * hidden, dim), base + 2)
        wd = normal((dim, hidden), base + 3)
        if tp_ranks == 1:
            keep["wq"].append(wqkv)           # fused rows: q, k, v
            keep["wk"].append(None)
            keep["wv"].append(None)
            keep["wo"].append(wo)
            keep["w_gate"].append(wgu)        # gate rows then up rows
            keep["w_up"].append(None)
            keep["w_down"].append(wd)
        else:
            keep["wq"].append(rows(wqkv, sl["q_rows"]))
            keep["wk"].append(rows(wqkv, sl["k_rows"]))
            keep["wv"].append(rows(wqkv, sl["v_rows"]))
            keep["wo"].append(cols(wo, sl["wo_cols"]))
            keep["w_gate"].append(rows(wgu, sl["gate_rows"]))
            keep["w_up"].append(rows(wgu, sl["up_rows"]))
            keep["w_down"].append(cols(wd, sl["down_cols"]))
        keep["attn_norm"].append(ones(dim))
        keep["ffn_norm"].append(ones(dim))
        del wqkv, wo, wgu, wd
    embed = normal((vocab, dim), 1)
    lm_full = normal((vocab, dim), 2)
    lm_head = lm_full if tp_ranks == 1 else rows(lm_full, sl["vocab_rows"])
    del lm_full
    final_norm = ones(dim)
    cos_h, sin_h = rope_tables(max_seq, head_dim, theta)
    cos = torch.from_numpy(cos_h).to(dev)
    sin = torch.from_numpy(sin_h).to(dev)
    torch.cuda.synchronize()

    def ptrs(name):
        return [t.data_ptr() if t is not None else None for t in keep[name]]

    weights = dict(embed=embed.data_ptr(), attn_norm=ptrs("attn_norm"),
                   wq=ptrs("wq"), wk=ptrs("wk"), wv=ptrs("wv"),
                   wo=ptrs("wo"), ffn_norm=ptrs("ffn_norm"),
                   w_gate=ptrs("w_gate"), w_up=ptrs("w_up"),
                   w_down=ptrs("w_down"), final_norm=final_norm.data_ptr(),
                   lm_head=lm_head.data_ptr(), cos=cos.data_ptr(),
                   sin=sin.data_ptr())
    cfg = DecoderConfig(dim=dim, hidden=hidden, n_layers=n_layers,
                        q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                        vocab=vocab, max_seq=max_seq, eps=eps, rope_theta=theta,
                        weights_bf16=1, batch=batch, tp_ranks=tp_ranks,
                        tp_reduce=tp_reduce if tp_ranks > 1 else 0)
    tensors = dict(keep, embed=embed, lm_head=lm_head, final_norm=final_norm,
                   cos=cos_h, sin=sin_h)
    # The decoder reads the device tables for its whole life: hold them, or the
    # caching allocator hands their block to the next small allocation.
    return Decoder(cfg, weights, keep=(tensors, cos, sin)), tensors


def nn_quant_model(quant, dim, hidden, n_layers, q_heads, kv_heads, head_dim,
                   vocab, max_seq, seed=7, theta=10000.0, eps=1e-5):
    """The std::nn model with the four projections of every layer quantised on
    the GPU from the bf16 weights nn_bf16_model would make (quant "fp8" or
    "q4"); norms, embedding and classifier stay bf16. One sequence, one rank.
    Returns (Decoder, tensors)."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device())
    L = lib()
    code = 2 if quant == "fp8" else 3

    def normal(shape, tensor_id):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        rc = L.vx_b200_fill_normal(t.data_ptr(), 1, t.numel(),
                                   seed * 1000003 + tensor_id, 0.02)
        assert rc == 0, L.vx_b200_last_error()
        return t

    def quantised(w):
        rows, cols = w.shape
        if quant == "fp8":
            codes = torch.empty(rows * cols, dtype=torch.uint8, device=dev)
            scales = torch.empty(((rows + 127) // 128) * (cols // 128),
                                 dtype=torch.float32, device=dev)
        else:
            codes = torch.empty(rows * cols // 2, dtype=torch.uint8, device=dev)
            scales = torch.empty(rows * (cols // 32), dtype=torch.float16,
                                 device=dev)
        rc = L.vx_b200_quantize(code, w.data_ptr(), rows, cols, codes.data_ptr(),
                                scales.data_ptr())
        assert rc == 0, L.vx_b200_last_error()
        return codes.view(torch.int32), scales

    keep = {k: [] for k in ("attn_norm", "wq", "s_qkv", "wo", "s_o", "ffn_norm",
                            "w_gate", "s_gate_up", "w_down", "s_down")}
    for l in range(n_layers):
        base = 16 * (l + 1)
        for name, sname, shape, tid in (
                ("wq", "s_qkv", ((q_heads + 2 * kv_heads) * head_dim, dim), 0),
                ("wo", "s_o", (dim, q_heads * head_dim), 1),
                ("w_gate", "s_gate_up", (2 * hidden, dim), 2),
                ("w_down", "s_down", (dim, hidden), 3)):
            w = normal(shape, base + tid)
            codes, scales = quantised(w)
            torch.cuda.synchronize()
            del w
            keep[name].append(codes)
            keep[sname].append(scales)
        keep["attn_norm"].append(torch.ones(dim, dtype=torch.bfloat16, device=dev))
        keep["ffn_norm"].append(torch.ones(dim, dtype=torch.bfloat16, device=dev))
    embed = normal((vocab, dim), 1)
    lm_head = normal((vocab, dim), 2)
    final_norm = torch.ones(dim, dtype=torch.bfloat16, device=dev)
    cos_h, sin_h = rope_tables(max_seq, head_dim, theta)
    cos = torch.from_numpy(cos_h).to(dev)
    sin = torch.from_numpy(sin_h).to(dev)
    torch.cuda.synchronize()

    def ptrs(name):
        return [t.data_ptr() for t in keep[name]]

    nothing = [None] * n_layers
    weights = dict(embed=embed.data_ptr(), attn_norm=ptrs("attn_norm"),
                   wq=ptrs("wq"), wk=nothing, wv=nothing, wo=ptrs("wo"),
                   ffn_norm=ptrs("ffn_norm"), w_gate=ptrs("w_gate"), w_up=nothing,
                   w_down=ptrs("w_down"), final_norm=final_norm.data_ptr(),
                   lm_head=lm_head.data_ptr(), cos=cos.data_ptr(),
                   sin=sin.data_ptr(), s_qkv=ptrs("s_qkv"), s_o=ptrs("s_o"),
                   s_gate_up=ptrs("s_gate_up"), s_down=ptrs("s_down"))
    cfg = DecoderConfig(dim=dim, hidden=hidden, n_layers=n_layers,
                        q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                        vocab=vocab, max_seq=max_seq, eps=eps, rope_theta=theta,
                        weights_bf16=code, batch=1, tp_ranks=1, tp_reduce=0)
    tensors = dict(keep, embed=embed, lm_head=lm_head, final_norm=final_norm,
                   cos=cos_h, sin=sin_h)
    # The decoder reads the device tables for its whole life: hold them, or the
    # caching allocator hands their block to the next small allocation.
    return Decoder(cfg, weights, keep=(tensors, cos, sin)), tensors


LLAMA2_7B = dict(dim=4096, hidden=11008, n_layers=32, q_heads=32, kv_heads=32,
                 head_dim=128, vocab=32000)


def weight_bytes_per_token(dim, hidden, n_layers, q_heads, kv_heads, head_dim,
                           vocab, elem_bytes=2):
    """Bytes of weights one decode step streams (every matrix once, the
    classifier included, one embedding row not counted)."""
    per_layer = ((q_heads + 2 * kv_heads) * head_dim * dim
                 + dim * q_heads * head_dim + 3 * dim * hidden)
    return (n_layers * per_layer + vocab * dim) * elem_bytes
