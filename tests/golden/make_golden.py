"""Regenerates tests/golden/oracle_golden.json from the CPU oracle.

The reference ships no golden vectors for this path (its comparisons are made at run time
against MLX on an Apple GPU), so these vectors are produced by the oracle itself: they pin the
oracle -- generator, quantiser, canonical GEMV, router, a greedy token stream -- against
accidental change, and let the GPU tests check fixed values without running the oracle.
Run:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def compute():
    from oracle import oracle as O
    from conftest import TINY, SEED, JITTER, CONV_STD
    out = {}
    out["tokens_seed5"] = [int(t) for t in O.synth_tokens(5, "prompt", 8, 151936)]
    out["f16_seed0_x"] = [int(v) for v in O.synth_f16(0, "x", 8).view(np.uint16)]
    p, s, b = O.synth_q4(0, "cfg1.w", 4096, 2048)
    out["cfg1_w_sha"] = [sha(p), sha(s), sha(b)]
    out["cfg1_w_row0"] = [int(v) for v in p[0, :4]] + [int(v) for v in s[0, :2].view(np.uint16)] + [int(v) for v in b[0, :2].view(np.uint16)]
    for M in (1, 8):
        x = O.synth_f16(0, "cfg1.x", M * 2048, 0.0, 1.0).reshape(M, 2048)
        y = O.qmm4(x, p, s, b)
        out[f"cfg1_y_M{M}_sha"] = sha(y)
        out[f"cfg1_y_M{M}_head"] = [int(v) for v in y[0, :8].view(np.uint16)]
    logits = O.synth_f16(2, "router.logits", 4 * 256).reshape(4, 256)
    inds, scores = O.route_topk(logits, 8)
    out["route_inds"] = inds.tolist()
    out["route_scores"] = [int(v) for v in scores.reshape(-1).view(np.uint16)]
    cfg = O.config(norm_jitter=JITTER, conv_std=CONV_STD, **TINY)
    m = O.Model(cfg, SEED)
    st = m.stream(64)
    prompt = O.synth_tokens(SEED, "golden.prompt", 6, cfg.vocab)
    toks = [int(st.step(prompt)[-1])]
    for _ in range(9):
        toks.append(int(st.step([toks[-1]])[0]))
    out["tiny_greedy"] = toks
    out["tiny_blob_sha"] = sha(st.state_save())
    # speculative-sampling rows: draws, draft-excluded draws and accept flags at two settings
    sl = O.synth_f16(5, "sampler.logits", 4 * 2048, 0.0, 2.5).reshape(4, 2048)
    draft = np.array([3, -1, 100, 5], dtype=np.int32)
    for name, inv_t, top_p in (("sample_t0p7", 1.0 / 0.7, 1.0), ("sample_nucleus", 1.0, 0.9)):
        f, r, a = O.sample_rows(sl, draft, inv_t, top_p, 0x1234, 0xABCD, 40)
        out[name] = [f.tolist(), r.tolist(), a.tolist()]
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "oracle_golden.json"), "w") as f:
        json.dump(compute(), f, indent=1, sort_keys=True)
    print("written")
