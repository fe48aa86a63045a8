"""ctypes binding of the CPU oracle (oracle/seedless_oracle.cpp).

Test infrastructure only: imported by tests/, the smoke check and the CPU-baseline legs of
bench.py.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libseedless_oracle.so")


def build(force=False):
    """Compile the oracle with the Makefile beside it (g++ only)."""
    src = os.path.join(_HERE, "seedless_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


class OrcConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("n_layers", C.c_int32), ("attn_every", C.c_int32), ("vocab", C.c_int32),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("moe_inter", C.c_int32),
        ("gdn_k_heads", C.c_int32), ("gdn_v_heads", C.c_int32),
        ("attn_heads", C.c_int32), ("attn_kv_heads", C.c_int32),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float),
        ("norm_jitter", C.c_float), ("conv_std", C.c_float),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_tensor_seed.restype = C.c_uint64
        L.orc_tensor_seed.argtypes = [C.c_uint64, C.c_char_p]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.POINTER(OrcConfig), C.c_uint64]
        L.orc_model_create_lazy.restype = C.c_void_p
        L.orc_model_create_lazy.argtypes = [C.POINTER(OrcConfig), C.c_uint64]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_model_tensor.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]
        L.orc_model_tensor_count.argtypes = [C.c_void_p]
        L.orc_model_tensor_name.restype = C.c_char_p
        L.orc_model_tensor_name.argtypes = [C.c_void_p, C.c_int]
        L.orc_stream_create.restype = C.c_void_p
        L.orc_stream_create.argtypes = [C.c_void_p, C.c_int]
        L.orc_stream_destroy.argtypes = [C.c_void_p]
        L.orc_stream_len.argtypes = [C.c_void_p]
        L.orc_state_size.restype = C.c_uint64
        L.orc_state_size.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def tensor_seed(base_seed, name):
    return lib().orc_tensor_seed(C.c_uint64(base_seed), name.encode())


def synth_f16(base_seed, name, n, mean=0.0, std=1.0):
    out = np.empty(n, dtype=np.float16)
    lib().orc_synth_f16(C.c_uint64(tensor_seed(base_seed, name)), C.c_uint64(n), C.c_float(mean), C.c_float(std), _p(out))
    return out


def synth_f32(base_seed, name, n, mean=0.0, std=1.0):
    out = np.empty(n, dtype=np.float32)
    lib().orc_synth_f32(C.c_uint64(tensor_seed(base_seed, name)), C.c_uint64(n), C.c_float(mean), C.c_float(std), _p(out))
    return out


def synth_tokens(base_seed, name, n, vocab):
    out = np.empty(n, dtype=np.int32)
    lib().orc_synth_tokens(C.c_uint64(tensor_seed(base_seed, name)), C.c_uint64(n), C.c_int32(vocab), _p(out))
    return out


def quantize_q4(w):
    """w fp16 [N,K] -> (packed u32 [N,K/8], scales fp16 [N,K/64], biases fp16 [N,K/64])."""
    w = np.ascontiguousarray(w, dtype=np.float16)
    N, K = w.shape
    packed = np.empty((N, K // 8), dtype=np.uint32)
    s = np.empty((N, K // 64), dtype=np.float16)
    b = np.empty((N, K // 64), dtype=np.float16)
    lib().orc_quantize_q4(_p(w), C.c_int64(N), C.c_int64(K), _p(packed), _p(s), _p(b))
    return packed, s, b


def synth_q4(base_seed, name, N, K, std=0.02):
    packed = np.empty((N, K // 8), dtype=np.uint32)
    s = np.empty((N, K // 64), dtype=np.float16)
    b = np.empty((N, K // 64), dtype=np.float16)
    lib().orc_synth_q4(C.c_uint64(tensor_seed(base_seed, name)), C.c_int64(N), C.c_int64(K), C.c_float(std), _p(packed), _p(s), _p(b))
    return packed, s, b


def dequant_q4(packed, s, b):
    N, K8 = packed.shape
    out = np.empty((N, K8 * 8), dtype=np.float32)
    lib().orc_dequant_q4(_p(packed), _p(s), _p(b), C.c_int64(N), C.c_int64(K8 * 8), _p(out))
    return out


def dequant_q4_half(packed, s, b):
    """fp16 rows of a 4-bit table, the reference's embed_rows_q4 arithmetic (SeedlessFusedVerify.swift:556-570)."""
    N, K8 = packed.shape
    out = np.empty((N, K8 * 8), dtype=np.float16)
    lib().orc_dequant_q4_half(_p(np.ascontiguousarray(packed)), _p(np.ascontiguousarray(s)), _p(np.ascontiguousarray(b)),
                              C.c_int64(N), C.c_int64(K8 * 8), _p(out))
    return out


def qmm8(x, w8, s, b):
    """8-bit group-64 GEMV (qmm8, SeedlessMetalForward.swift:384-434); w8 uint8 [N,K]."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, K = x.shape
    N = w8.shape[0]
    y = np.empty((M, N), dtype=np.float16)
    lib().orc_qmm8(_p(x), _p(np.ascontiguousarray(w8)), _p(np.ascontiguousarray(s)), _p(np.ascontiguousarray(b)),
                   C.c_int(M), C.c_int(K), C.c_int(N), _p(y))
    return y


def quantize_q8(w):
    """fp16 [N,K] -> (uint8 [N,K], fp16 scales [N,K/64], fp16 biases [N,K/64]): affine 8-bit per group of 64
    (test input maker; any bytes / scales / biases are valid input to qmm8)."""
    w = np.asarray(w, dtype=np.float32)
    N, K = w.shape
    g = w.reshape(N, K // 64, 64)
    lo, hi = g.min(axis=2), g.max(axis=2)
    scale = np.maximum((hi - lo) / 255.0, 1e-7).astype(np.float16)
    bias = lo.astype(np.float16)
    q = np.clip(np.rint((g - bias.astype(np.float32)[:, :, None]) / scale.astype(np.float32)[:, :, None]), 0, 255).astype(np.uint8)
    return q.reshape(N, K), scale, bias


def set_num_threads(n):
    """OpenMP threads of the oracle's loops; returns the count in force."""
    lib().orc_set_num_threads.restype = C.c_int
    return int(lib().orc_set_num_threads(C.c_int(int(n))))


def qmm4(x, packed, s, b):
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, K = x.shape
    N = packed.shape[0]
    y = np.empty((M, N), dtype=np.float16)
    lib().orc_qmm4(_p(x), _p(packed), _p(s), _p(b), C.c_int(M), C.c_int(K), C.c_int(N), _p(y))
    return y


def fmm(x, w):
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(w, dtype=np.float16)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), dtype=np.float16)
    lib().orc_fmm(_p(x), _p(w), C.c_int(M), C.c_int(K), C.c_int(N), _p(y))
    return y


def rmsnorm(x, w, eps=1e-6):
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, D = x.shape
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), C.c_int(M), C.c_int(D), C.c_float(eps), _p(out))
    return out


def route_topk(logits, topk=8):
    logits = np.ascontiguousarray(logits, dtype=np.float16)
    M, E = logits.shape
    inds = np.empty((M, topk), dtype=np.int32)
    scores = np.empty((M, topk), dtype=np.float16)
    lib().orc_route_topk(_p(logits), C.c_int(M), C.c_int(E), C.c_int(topk), _p(inds), _p(scores))
    return inds, scores


class Model:
    """Synthetic model generated from (config, seed); tensors are readable by name."""

    def __init__(self, cfg: OrcConfig, seed: int, lazy_experts: bool = False):
        self.cfg = cfg
        self.seed = seed
        make = lib().orc_model_create_lazy if lazy_experts else lib().orc_model_create
        self.h = make(C.byref(cfg), C.c_uint64(seed))

    def set_gdn_norm_f32(self, layer, w):
        """Give one GDN layer an f32 norm weight (the reference then keeps the normed value in f32)."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        assert w.size == 128 and lib().orc_model_set_gdn_norm_f32(C.c_void_p(self.h), C.c_int(layer), _p(w)) == 0

    def set_router_q8(self, layer, rw, rs, rb, gw, gs, gb):
        """Give one layer its router / shared gate in the checkpoint's 8-bit group-64 layout."""
        keep = [np.ascontiguousarray(a) for a in (rw, rs, rb, gw, gs, gb)]
        rc = lib().orc_model_set_router_q8(C.c_void_p(self.h), C.c_int(layer), *[_p(a) for a in keep])
        assert rc == 0

    def close(self):
        if self.h:
            lib().orc_model_destroy(C.c_void_p(self.h))
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor_names(self):
        n = lib().orc_model_tensor_count(C.c_void_p(self.h))
        return [lib().orc_model_tensor_name(C.c_void_p(self.h), i).decode() for i in range(n)]

    def tensor_bytes(self, name):
        ptr = C.c_void_p()
        nb = C.c_uint64()
        rc = lib().orc_model_tensor(C.c_void_p(self.h), name.encode(), C.byref(ptr), C.byref(nb))
        if rc != 0:
            raise KeyError(name)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(nb.value,))

    def moe_block(self, layer, x):
        x = np.ascontiguousarray(x, dtype=np.float16)
        M = x.shape[0]
        out = np.empty_like(x)
        inds = np.empty((M, self.cfg.top_k), dtype=np.int32)
        scores = np.empty((M, self.cfg.top_k), dtype=np.float16)
        lib().orc_moe_block(C.c_void_p(self.h), C.c_int(layer), _p(x), C.c_int(M), _p(out), _p(inds), _p(scores))
        return out, inds, scores

    def lm_head(self, normed):
        normed = np.ascontiguousarray(normed, dtype=np.float16)
        M = normed.shape[0]
        logits = np.empty((M, self.cfg.vocab), dtype=np.float16)
        toks = np.empty(M, dtype=np.int32)
        lib().orc_lm_head(C.c_void_p(self.h), _p(normed), C.c_int(M), _p(logits), _p(toks))
        return logits, toks

    def embed(self, tokens):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((len(tokens), self.cfg.hidden), dtype=np.float16)
        lib().orc_embed(C.c_void_p(self.h), _p(tokens), C.c_int(len(tokens)), _p(out))
        return out

    def head(self, h):
        h = np.ascontiguousarray(h, dtype=np.float16)
        M = h.shape[0]
        logits = np.empty((M, self.cfg.vocab), dtype=np.float16)
        toks = np.empty(M, dtype=np.int32)
        lib().orc_head(C.c_void_p(self.h), _p(h), C.c_int(M), _p(logits), _p(toks))
        return logits, toks

    def stream(self, max_seq_len):
        return Stream(self, max_seq_len)


class Stream:
    def __init__(self, model: Model, max_seq_len: int):
        self.model = model
        self.h = lib().orc_stream_create(C.c_void_p(model.h), C.c_int(max_seq_len))

    def close(self):
        if self.h:
            lib().orc_stream_destroy(C.c_void_p(self.h))
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def length(self):
        return lib().orc_stream_len(C.c_void_p(self.h))

    def set_length(self, n):
        if lib().orc_stream_set_len(C.c_void_p(self.h), C.c_int(n)) != 0:
            raise ValueError("length out of range")

    def forward(self, tokens):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((len(tokens), self.model.cfg.hidden), dtype=np.float16)
        rc = lib().orc_forward(C.c_void_p(self.h), _p(tokens), C.c_int(len(tokens)), _p(out))
        if rc != 0:
            raise RuntimeError(f"orc_forward rc={rc}")
        return out

    def step(self, tokens, want_logits=False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        M = len(tokens)
        logits = np.empty((M, self.model.cfg.vocab), dtype=np.float16) if want_logits else None
        out = np.empty(M, dtype=np.int32)
        rc = lib().orc_step(C.c_void_p(self.h), _p(tokens), C.c_int(M), _p(logits), _p(out))
        if rc != 0:
            raise RuntimeError(f"orc_step rc={rc}")
        return (out, logits) if want_logits else out

    def mixer_rows(self, layer, x, pos0):
        x = np.ascontiguousarray(x, dtype=np.float16)
        out = np.empty_like(x)
        rc = lib().orc_mixer_rows(C.c_void_p(self.h), C.c_int(layer), _p(x), C.c_int(x.shape[0]), C.c_int(pos0), _p(out))
        if rc != 0:
            raise RuntimeError(f"orc_mixer_rows rc={rc}")
        return out

    def layer_rows(self, layer, h_in, pos0):
        h_in = np.ascontiguousarray(h_in, dtype=np.float16)
        out = np.empty_like(h_in)
        rc = lib().orc_layer_rows(C.c_void_p(self.h), C.c_int(layer), _p(h_in), C.c_int(h_in.shape[0]), C.c_int(pos0), _p(out))
        if rc != 0:
            raise RuntimeError(f"orc_layer_rows rc={rc}")
        return out

    def state_save(self):
        n = lib().orc_state_size(C.c_void_p(self.h))
        buf = np.empty(n, dtype=np.uint8)
        rc = lib().orc_state_save(C.c_void_p(self.h), _p(buf), C.c_uint64(n))
        if rc != 0:
            raise RuntimeError("orc_state_save failed")
        return buf

    def state_restore(self, blob):
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        return lib().orc_state_restore(C.c_void_p(self.h), _p(blob), C.c_uint64(len(blob))) == 0


def set_alt_order(on):
    """Control experiment only: use another (equally valid) lane-reduction order."""
    lib().orc_set_alt_order(C.c_int(1 if on else 0))


def config(hidden=2048, n_layers=40, attn_every=4, vocab=151936, n_experts=256, top_k=8, moe_inter=512,
           gdn_k_heads=16, gdn_v_heads=32, attn_heads=16, attn_kv_heads=2, rope_theta=1e7, rms_eps=1e-6,
           norm_jitter=0.0, conv_std=0.02):
    return OrcConfig(hidden, n_layers, attn_every, vocab, n_experts, top_k, moe_inter, gdn_k_heads, gdn_v_heads,
                     attn_heads, attn_kv_heads, rope_theta, rms_eps, norm_jitter, conv_std)


def sample_rows(logits, draft, inv_t, top_p, seed_lo, seed_hi, base_pos, logit_adj=None):
    """CPU restatement of the speculative-sampling rows: -> (full, resid, accept) int32 [M].
    logit_adj: optional f32 [V] added to every row's logits first."""
    logits = np.ascontiguousarray(logits, dtype=np.float16)
    M, V = logits.shape
    d = None if draft is None else np.ascontiguousarray(draft, dtype=np.int32)
    adj = None if logit_adj is None else np.ascontiguousarray(logit_adj, dtype=np.float32)
    full, resid, acc = (np.empty(M, dtype=np.int32) for _ in range(3))
    lib().orc_sample_rows(_p(logits), _p(adj) if adj is not None else None, C.c_int(M), C.c_int(V), _p(d) if d is not None else None, C.c_float(inv_t), C.c_float(top_p),
                          C.c_uint32(seed_lo), C.c_uint32(seed_hi), C.c_uint32(base_pos), _p(full), _p(resid), _p(acc))
    return full, resid, acc
