"""Checkpoint intake (host logic): the reference's tensor names (SeedlessEngine.swift:33-143) mapped to
this library's, read from a safetensors file written here from the CPU restatement's tensors."""
import os

import numpy as np
import pytest

from conftest import SEED, TINY, oracle_model


def fake_checkpoint(path, model, geom):
    """Write the oracle model's tensors under the checkpoint's names; the embedding as a 4-bit table, the
    router / shared gate 8-bit, layer 0's GDN norm weight as f32 (the case the reference promotes).  Returns the
    dict the loader is expected to give back."""
    from oracle import oracle as O
    from qwisp_b200 import checkpoint as CK
    H, E, V = geom["hidden"], geom["n_experts"], geom["vocab"]
    want = {n: model.tensor_bytes(n).copy() for n in model.tensor_names()}
    want.pop("embed")
    ew, es, eb = O.synth_q4(SEED, "ckpt.embed", V, H)
    want.update({"embed.w": ew, "embed.s": es, "embed.b": eb})
    for i in range(geom["n_layers"]):
        r16 = want.pop(f"L{i}.moe.router").view(np.float16).reshape(E, H)
        g16 = want.pop(f"L{i}.moe.shared_gate").view(np.float16).reshape(1, H)
        for nm, src in ((f"L{i}.moe.router", r16), (f"L{i}.moe.shared_gate", g16)):
            w8, s, b = O.quantize_q8(src)
            want.update({nm + ".w": w8, nm + ".s": s, nm + ".b": b})
    file = {}
    for dst, src in CK.name_map(geom["n_layers"], geom["attn_every"]).items():
        a = np.ascontiguousarray(want[dst]).reshape(-1)
        if dst.endswith((".gdn.conv_w", ".gdn.A_log", ".gdn.dt_bias")):
            a = a.view(np.uint8).view(np.float32)
            if dst.endswith("conv_w"):
                a = a.reshape(-1, 4, 1)
        elif dst == "L0.gdn.norm":                               # stored f32: handed on as f32 (the promoted norm)
            a = a.view(np.uint8).view(np.float16).astype(np.float32)
            want.pop(dst); want[dst + ".f32"] = a.copy()
        elif dst.endswith(".w"):
            a = a.view(np.uint8).view(np.uint32)
        else:
            a = a.view(np.uint8).view(np.float16)
        file[src] = a
    CK.write_safetensors(path, file)
    return want


def test_name_map_covers_the_reference_table():
    from qwisp_b200 import checkpoint as CK
    m = CK.name_map(40, 4)
    assert len(set(m.values())) == len(m)
    assert m["embed.w"] == "language_model.model.embed_tokens.weight"
    assert m["lm_head.s"] == "language_model.lm_head.scales"
    assert m["L3.attn.q_proj.w"] == "language_model.model.layers.3.self_attn.q_proj.weight"
    assert m["L0.gdn.in_proj_qkv.b"] == "language_model.model.layers.0.linear_attn.in_proj_qkv.biases"
    assert m["L0.moe.router.w"] == "language_model.model.layers.0.mlp.gate.weight"
    assert m["L0.moe.shared_gate.s"] == "language_model.model.layers.0.mlp.shared_expert_gate.scales"
    assert m["L0.moe.shared_down_proj.w"] == "language_model.model.layers.0.mlp.shared_expert.down_proj.weight"
    assert "L3.gdn.conv_w" not in m and "L0.attn.q_norm" not in m       # 3 GDN : 1 attention
    # per GDN layer 15 q4 + 4 plain, per attention layer 12 + 2, every layer 2 norms + 6 + 18 MoE tensors
    assert len(m) == 3 + 1 + 3 + 30 * (19 + 26) + 10 * (14 + 26)


def test_checkpoint_roundtrip(tmp_path):
    from qwisp_b200 import checkpoint as CK
    model = oracle_model(TINY)
    path = os.path.join(tmp_path, "tiny.safetensors")
    want = fake_checkpoint(path, model, TINY)
    got = CK.load_checkpoint(path, TINY["n_layers"], TINY["attn_every"])
    assert set(got) == set(want)
    for n in want:
        assert np.array_equal(np.ascontiguousarray(got[n]).view(np.uint8).reshape(-1), np.ascontiguousarray(want[n]).view(np.uint8).reshape(-1)), n
    assert got["L0.gdn.conv_w"].dtype == np.float32 and got["L0.gdn.norm.f32"].dtype == np.float32 and got["L1.in_norm"].dtype == np.float16
    # a missing tensor is named, like the reference's store.req
    raw = {k: v[0] for k, v in CK.read_safetensors(path).items()}
    raw.pop("language_model.model.norm.weight")
    short = os.path.join(tmp_path, "short.safetensors")
    CK.write_safetensors(short, raw)
    with pytest.raises(KeyError, match="language_model.model.norm.weight"):
        CK.load_checkpoint(short, TINY["n_layers"], TINY["attn_every"])
    model.close()


def test_bf16_plain_tensors_are_widened():
    from qwisp_b200 import checkpoint as CK
    bits = np.array([0x3F80, 0xC000, 0x3DCD], dtype=np.uint16)           # 1.0, -2.0, ~0.1
    f = CK._as_f32(bits, "BF16")
    assert f[0] == 1.0 and f[1] == -2.0 and abs(f[2] - 0.1) < 1e-3


@pytest.mark.gpu
def test_engine_from_checkpoint(tmp_path):
    import qwisp_b200 as Q
    from oracle import oracle as O
    model = oracle_model(TINY)
    path = os.path.join(tmp_path, "tiny.safetensors")
    want = fake_checkpoint(path, model, TINY)
    cfg = Q.config(**TINY, max_rows=16, max_streams=2, kv_page_size=32, kv_pages=8)
    a, b = Q.Engine.from_checkpoint(cfg, path), Q.Engine.from_tensors(cfg, want)
    try:
        p = O.synth_tokens(SEED, "ckpt", 7, TINY["vocab"])
        la, lb = a.stream(32).step_logits(p), b.stream(32).step_logits(p)
        assert np.isfinite(la.astype(np.float32)).all()
        assert np.array_equal(la.view(np.uint16), lb.view(np.uint16))
    finally:
        a.close(); b.close(); model.close()
