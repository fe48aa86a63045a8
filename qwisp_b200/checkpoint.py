"""Checkpoint intake: safetensors files in the reference's tensor naming -> the tensor names of
`include/seedless_b200.h`.

The reference builds its engine from a `WeightStore` by name
(`swift/Sources/QwispCore/SeedlessEngine.swift:33-144`): `language_model.model.layers.<i>.…` with
`.weight/.scales/.biases` triples in the MLX affine layout.  `name_map` restates that table for this
library's names; nothing is re-quantised: 4-bit tensors, the 4-bit embedding and the 8-bit router /
shared-expert gate go to the engine in the layout they are stored in.  Only the small plain tensors
are cast (`conv1d.weight`, `A_log`, `dt_bias` to f32; norm weights to f16, except a GDN norm weight
stored as f32, which is handed over as f32 so that norm runs in f32 as in the reference).

The safetensors container (8-byte little-endian header length, a JSON header with dtype / shape /
data_offsets per tensor, then the raw bytes) is read here with numpy only.
"""
import json
import struct

import numpy as np

_DTYPES = {"F16": np.float16, "F32": np.float32, "F64": np.float64, "U8": np.uint8, "I8": np.int8,
           "U16": np.uint16, "I16": np.int16, "U32": np.uint32, "I32": np.int32, "U64": np.uint64, "I64": np.int64,
           "BF16": np.uint16}      # bf16 is kept as its bit pattern; see _as_f32
_NAMES = {np.dtype(v).name: k for k, v in _DTYPES.items() if k != "BF16"}

_ROOT = "language_model.model"
_Q = (("weight", "w"), ("scales", "s"), ("biases", "b"))


def is_attention_layer(i, attn_every):
    """SeedlessEngine.isLinear (SeedlessEngine.swift:29) negated."""
    return (i + 1) % attn_every == 0


def name_map(n_layers, attn_every):
    """dict: this library's tensor name -> the checkpoint's tensor name (SeedlessEngine.swift:33-143)."""
    m = {}

    def q(dst, src):
        for long, short in _Q:
            m[f"{dst}.{short}"] = f"{src}.{long}"

    q("embed", f"{_ROOT}.embed_tokens")
    m["final_norm"] = f"{_ROOT}.norm.weight"
    q("lm_head", "language_model.lm_head")
    for i in range(n_layers):
        p, d = f"{_ROOT}.layers.{i}", f"L{i}"
        m[f"{d}.in_norm"] = f"{p}.input_layernorm.weight"
        m[f"{d}.post_norm"] = f"{p}.post_attention_layernorm.weight"
        if is_attention_layer(i, attn_every):
            for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
                q(f"{d}.attn.{proj}", f"{p}.self_attn.{proj}")
            m[f"{d}.attn.q_norm"] = f"{p}.self_attn.q_norm.weight"
            m[f"{d}.attn.k_norm"] = f"{p}.self_attn.k_norm.weight"
        else:
            for proj in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj"):
                q(f"{d}.gdn.{proj}", f"{p}.linear_attn.{proj}")
            m[f"{d}.gdn.conv_w"] = f"{p}.linear_attn.conv1d.weight"
            m[f"{d}.gdn.norm"] = f"{p}.linear_attn.norm.weight"
            m[f"{d}.gdn.A_log"] = f"{p}.linear_attn.A_log"
            m[f"{d}.gdn.dt_bias"] = f"{p}.linear_attn.dt_bias"
        q(f"{d}.moe.router", f"{p}.mlp.gate")                       # 8-bit group-64
        q(f"{d}.moe.shared_gate", f"{p}.mlp.shared_expert_gate")    # 8-bit group-64, one row
        for proj in ("gate_proj", "up_proj", "down_proj"):
            q(f"{d}.moe.{proj}", f"{p}.mlp.switch_mlp.{proj}")
            q(f"{d}.moe.shared_{proj}", f"{p}.mlp.shared_expert.{proj}")
    return m


_F32 = (".gdn.conv_w", ".gdn.A_log", ".gdn.dt_bias")
_F16 = ("final_norm", ".in_norm", ".post_norm", ".gdn.norm", ".attn.q_norm", ".attn.k_norm")


def _as_f32(arr, st_dtype):
    if st_dtype == "BF16":
        return (arr.astype(np.uint32) << 16).view(np.float32)
    return arr.astype(np.float32)


def read_safetensors(path):
    """dict: name -> (numpy array over a memory map of the file, safetensors dtype string)."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen <= 0 or hlen > (100 << 20):
            raise ValueError(f"{path}: implausible safetensors header length {hlen}")
        header = json.loads(f.read(hlen).decode("utf-8"))
    raw = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen)
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = info["dtype"]
        if dt not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
        b, e = info["data_offsets"]
        npdt = np.dtype(_DTYPES[dt])
        shape = tuple(info["shape"])
        if b < 0 or e > raw.size or (e - b) != int(np.prod(shape, dtype=np.int64)) * npdt.itemsize:
            raise ValueError(f"{path}: tensor {name} has inconsistent offsets / shape")
        out[name] = (raw[b:e].view(npdt).reshape(shape), dt)
    return out


def write_safetensors(path, tensors):
    """Write dict name -> numpy array (dtypes of _DTYPES except bf16) as one safetensors file."""
    header, off = {}, 0
    keep = {}
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr)
        keep[name] = a
        header[name] = {"dtype": _NAMES[a.dtype.name], "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in tensors:
            f.write(keep[name].tobytes())


def load_checkpoint(paths, n_layers, attn_every):
    """Read the safetensors shards and return dict: this library's tensor name -> contiguous numpy array,
    ready for `Engine.from_tensors`.  Raises KeyError naming the first tensor the reference's table
    requires (`store.req`, SeedlessEngine.swift:40-143) that no shard holds."""
    if isinstance(paths, (str, bytes)):
        paths = [paths]
    store = {}
    for p in paths:
        store.update(read_safetensors(p))
    out = {}
    for dst, src in name_map(n_layers, attn_every).items():
        if src not in store:
            raise KeyError(src)
        arr, dt = store[src]
        if dst.endswith(".gdn.norm") and dt == "F32":     # the reference promotes this norm to f32 (SeedlessFusedVerify.swift:2815-2818)
            out[dst + ".f32"] = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
            continue
        if dst.endswith(_F32):
            arr = _as_f32(arr, dt)                      # conv1d.weight [C,K,1] -> f32 [C,K] (same order)
        elif dst.endswith(_F16):
            arr = _as_f32(arr, dt).astype(np.float16) if dt != "F16" else arr
        elif dst.endswith((".s", ".b")) and dt != "F16":
            arr = _as_f32(arr, dt).astype(np.float16)
        out[dst] = np.ascontiguousarray(arr).reshape(-1)
    return out
