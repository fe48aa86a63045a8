"""Single operators over the C ABI -- the counterparts of the reference's per-op wrappers
its kernel tests call (SeedlessMetalForward.qmm, routeTop8Rows, moeBlockRows, gdnLayerRows,
attnLayerRows: swift/Sources/QwispCore/SeedlessMetalForward.swift:222,
SeedlessVerifyForward.swift:37-248)."""
import ctypes as C

import numpy as np

from ._lib import SeedlessError, lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def qmm4(x, packed, scales, biases):
    x = np.ascontiguousarray(x, dtype=np.float16)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    biases = np.ascontiguousarray(biases, dtype=np.float16)
    M, K = x.shape
    N = packed.shape[0]
    y = np.empty((M, N), dtype=np.float16)
    rc = lib().sl_op_qmm4(_p(x), _p(packed), _p(scales), _p(biases), M, K, N, _p(y))
    if rc != 0:
        raise SeedlessError(rc, "sl_op_qmm4")
    return y


def quantize_q4(w):
    w = np.ascontiguousarray(w, dtype=np.float16)
    N, K = w.shape
    packed = np.empty((N, K // 8), dtype=np.uint32)
    s = np.empty((N, K // 64), dtype=np.float16)
    b = np.empty((N, K // 64), dtype=np.float16)
    rc = lib().sl_op_quantize_q4(_p(w), N, K, _p(packed), _p(s), _p(b))
    if rc != 0:
        raise SeedlessError(rc, "sl_op_quantize_q4")
    return packed, s, b


def moe_block(engine, layer, x):
    x = np.ascontiguousarray(x, dtype=np.float16)
    M = x.shape[0]
    out = np.empty_like(x)
    inds = np.empty((M, engine.cfg.top_k), dtype=np.int32)
    scores = np.empty((M, engine.cfg.top_k), dtype=np.float16)
    engine._check(lib().sl_op_moe_block(engine._h, layer, _p(x), M, _p(out), _p(inds), _p(scores)), "sl_op_moe_block")
    return out, inds, scores


def mixer(stream, layer, x, pos0):
    x = np.ascontiguousarray(x, dtype=np.float16)
    out = np.empty_like(x)
    stream.engine._check(lib().sl_op_mixer(stream._h, layer, _p(x), x.shape[0], pos0, _p(out)), "sl_op_mixer")
    return out


def read_kv(stream, layer_index, pos0, n):
    """Cached K (post-RoPE) and V of an attention layer at positions pos0..pos0+n-1: two fp16 [kv_heads, n, 256]."""
    cfg = stream.engine.cfg
    k = np.empty((cfg.attn_kv_heads, n, 256), dtype=np.float16)
    v = np.empty_like(k)
    stream.engine._check(lib().sl_op_read_kv(stream._h, layer_index, pos0, n, _p(k), _p(v)), "sl_op_read_kv")
    return k, v


def layer(stream, layer_index, h_in, pos0):
    h_in = np.ascontiguousarray(h_in, dtype=np.float16)
    out = np.empty_like(h_in)
    stream.engine._check(lib().sl_op_layer(stream._h, layer_index, _p(h_in), h_in.shape[0], pos0, _p(out)), "sl_op_layer")
    return out


def head(engine, h_rows, want_logits=True):
    h_rows = np.ascontiguousarray(h_rows, dtype=np.float16)
    M = h_rows.shape[0]
    logits = np.empty((M, engine.cfg.vocab), dtype=np.float16) if want_logits else None
    toks = np.empty(M, dtype=np.int32)
    engine._check(lib().sl_op_head(engine._h, _p(h_rows), M, _p(logits), _p(toks)), "sl_op_head")
    return logits, toks


def lm_head(engine, normed, want_logits=True):
    normed = np.ascontiguousarray(normed, dtype=np.float16)
    M = normed.shape[0]
    logits = np.empty((M, engine.cfg.vocab), dtype=np.float16) if want_logits else None
    toks = np.empty(M, dtype=np.int32)
    engine._check(lib().sl_op_lm_head(engine._h, _p(normed), M, _p(logits), _p(toks)), "sl_op_lm_head")
    return logits, toks


def synth_tokens(seed, name, n, vocab):
    out = np.empty(n, dtype=np.int32)
    rc = lib().sl_synth_tokens(seed, name.encode(), n, vocab, _p(out))
    if rc != 0:
        raise SeedlessError(rc, "sl_synth_tokens")
    return out


def synth_f16(seed, name, n, mean=0.0, std=1.0):
    out = np.empty(n, dtype=np.float16)
    rc = lib().sl_synth_f16(seed, name.encode(), n, mean, std, _p(out))
    if rc != 0:
        raise SeedlessError(rc, "sl_synth_f16")
    return out


def sample_rows(engine, logits, draft, inv_t, top_p, seed_lo, seed_hi, base_pos, logit_adj=None):
    """The sampling kernel on host logits [M, vocab] fp16 -> (full, resid, accept) int32 [M].
    logit_adj: optional f32 [vocab] added to every row first (penalties + bias)."""
    logits = np.ascontiguousarray(logits, dtype=np.float16)
    M = logits.shape[0]
    d = None if draft is None else np.ascontiguousarray(draft, dtype=np.int32)
    adj = None if logit_adj is None else np.ascontiguousarray(logit_adj, dtype=np.float32)
    full, resid, acc = (np.empty(M, dtype=np.int32) for _ in range(3))
    engine._check(lib().sl_op_sample_rows(engine._h, _p(logits), M, _p(d) if d is not None else None,
                                          _p(adj) if adj is not None else None, float(inv_t), float(top_p),
                                          int(seed_lo), int(seed_hi), int(base_pos), _p(full), _p(resid), _p(acc)), "sl_op_sample_rows")
    return full, resid, acc
