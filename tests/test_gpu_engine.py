"""GPU tests of the engine through the C ABI: token parity with the CPU oracle and the
reference's invariance suite (M-row == sequential, chained == stepped, one-step rollback ==
replay, full snapshot / restore, QWS1 across arena sizes, lane batch == solo, fault firewall)."""
import json
import os

import numpy as np
import pytest

from conftest import MINI, ROOT, SEED, TINY, f16_report, gpu_engine

pytestmark = pytest.mark.gpu


def prompt(vocab, n, name="prompt"):
    from oracle import oracle as O
    return O.synth_tokens(SEED, name, n, vocab)


def test_tiny_greedy_matches_golden_and_oracle(tiny_engine, tiny_oracle):
    g = json.load(open(os.path.join(ROOT, "tests", "golden", "oracle_golden.json")))
    V = TINY["vocab"]
    p = prompt(V, 6, "golden.prompt")
    so, sg = tiny_oracle.stream(64), tiny_engine.stream(64)
    # teacher-forced: feed the oracle's tokens, compare per-step argmax and logits
    feed = list(p)
    ref_toks = g["tiny_greedy"]
    lg = sg.step_logits(p)
    ro, rl = so.step(p, want_logits=True)
    rep = f16_report(lg, rl)
    print("tiny prefill logits", rep)
    assert rep["max_abs"] <= 2e-2, rep
    agree = 0
    cur = ref_toks[0]
    got_first = int(np.argmax(lg[-1].astype(np.float32)))
    agree += got_first == ref_toks[0]
    for k in range(1, 10):
        t = int(sg.step_argmax([cur])[0])
        agree += t == ref_toks[k]
        cur = ref_toks[k]
    print("teacher-forced agreement", agree, "/ 10")
    assert agree >= 9
    sg.close()


def test_mini_logits_within_tolerance(mini_engine, mini_oracle):
    V = MINI["vocab"]
    p = prompt(V, 12)
    so, sg = mini_oracle.stream(64), mini_engine.stream(64)
    rt, rl = so.step(p, want_logits=True)
    lg = sg.step_logits(p)
    rep = f16_report(lg, rl)
    print("mini logits", rep)
    assert rep["max_abs"] <= 2e-2, rep
    hid_o = mini_oracle.stream(64).forward(p)
    hid_g = mini_engine.stream(64).forward(p)
    rep_h = f16_report(hid_g, hid_o)
    print("mini hidden", rep_h)
    assert rep_h["max_abs"] <= 5e-2
    # greedy agreement where the oracle's top-1 / top-2 margin is clear
    srt = np.sort(rl.astype(np.float32), axis=1)
    clear = (srt[:, -1] - srt[:, -2]) > 4 * rep["max_abs"]
    got = np.argmax(lg.astype(np.float32), axis=1)
    assert np.array_equal(got[clear], rt[clear])
    sg.close()


@pytest.mark.parametrize("plan", [[1], [2], [9], [17], [9, 3], [41]])
def test_rows_equal_sequential(tiny_engine, plan):
    """verify_forward_rows_bitexact: an M-row step is bit-identical to M single-row steps,
    including the caches it leaves (checked through the tokens of two further steps)."""
    V = TINY["vocab"]
    toks = prompt(V, sum(plan) + 3, "rows")
    a, b = tiny_engine.stream(64), tiny_engine.stream(64)
    pos = 0
    for m in plan:
        la = a.step_logits(toks[pos:pos + m])
        lb = np.concatenate([b.step_logits(toks[pos + i:pos + i + 1]) for i in range(m)])
        assert np.array_equal(la.view(np.uint16), lb.view(np.uint16)), plan
        pos += m
    assert np.array_equal(a.state_save(), b.state_save())
    ta, tb = a.step_argmax(toks[pos:pos + 3]), b.step_argmax(toks[pos:pos + 3])
    assert np.array_equal(ta, tb)
    a.close(); b.close()


def test_many_row_kernels_equal_pass_kernels():
    """Calls with more than 8 rows run the many-row kernels (weights dequantised once per block of rows, experts
    without CTA-wide barriers); SL_FLAG_PASS_KERNELS walks the same rows in passes of 8 with the one-to-eight-row
    kernels.  Both must give the same bits: logits of a 37-row call, the state it leaves, and 12 lanes batched."""
    import qwisp_b200 as Q
    V = MINI["vocab"]
    ea, eb = gpu_engine(MINI), gpu_engine(MINI, flags=Q._lib.SL_FLAG_PASS_KERNELS)
    try:
        toks = prompt(V, 37 + 19, "manyrows")
        a, b = ea.stream(128), eb.stream(128)
        la, lb = a.step_logits(toks[:37]), b.step_logits(toks[:37])
        assert np.array_equal(la.view(np.uint16), lb.view(np.uint16))
        la, lb = a.step_logits(toks[37:]), b.step_logits(toks[37:])
        assert np.array_equal(la.view(np.uint16), lb.view(np.uint16))
        assert np.array_equal(a.state_save(), b.state_save())
        # 12 lanes with different histories, 3 batched steps
        lanes_a, lanes_b, cur_a, cur_b = [], [], [], []
        for i in range(12):
            p = prompt(V, 2 + (i * 5) % 11, f"manyrows.lane{i}")
            sa, sb = ea.stream(64), eb.stream(64)
            cur_a.append(int(sa.step_argmax(p)[-1])); cur_b.append(int(sb.step_argmax(p)[-1]))
            lanes_a.append(sa); lanes_b.append(sb)
        assert cur_a == cur_b
        for _ in range(3):
            cur_a = [int(t) for t in ea.batch_step_argmax(lanes_a, cur_a)]
            cur_b = [int(t) for t in eb.batch_step_argmax(lanes_b, cur_b)]
            assert cur_a == cur_b
        for sa, sb in zip(lanes_a, lanes_b):
            assert np.array_equal(sa.state_save(), sb.state_save())
        assert not ea.gpu_fault() and not eb.gpu_fault()
    finally:
        ea.close(); eb.close()


@pytest.mark.parametrize("K", [2, 3, 8])
def test_chained_equals_stepped(tiny_engine, K):
    V = TINY["vocab"]
    p = prompt(V, 5, "chain")
    a, b = tiny_engine.stream(64), tiny_engine.stream(64)
    fa, fb = int(a.step_argmax(p)[-1]), int(b.step_argmax(p)[-1])
    assert fa == fb
    chained = a.chained_step_argmax(fa, K)
    stepped, cur = [], fb
    for _ in range(K):
        cur = int(b.step_argmax([cur])[0]); stepped.append(cur)
    assert list(chained) == stepped
    # chain -> step -> chain interleave
    c2 = a.chained_step_argmax(int(chained[-1]), 2)
    s2, cur = [], stepped[-1]
    for _ in range(2):
        cur = int(b.step_argmax([cur])[0]); s2.append(cur)
    assert list(c2) == s2
    assert np.array_equal(a.state_save(), b.state_save())
    a.close(); b.close()


def test_reject_rollback_equals_replay(tiny_engine):
    """a3_reject_rollback_equiv: verify batch, partial reject, one-step rollback, replay of the
    accepted prefix == never having run the rejected rows."""
    V = TINY["vocab"]
    p = prompt(V, 7, "spec")
    a, b = tiny_engine.stream(64), tiny_engine.stream(64)
    a.step_argmax(p); b.step_argmax(p)
    drafts = prompt(V, 6, "drafts")
    snap = a.snapshot()
    a.step_argmax(drafts)                       # verify batch of 6 rows
    a.rollback(snap)                            # reject after 2 accepted
    a.forward(drafts[:2], want_hidden=False)
    b.forward(drafts[:2], want_hidden=False)
    assert a.length == b.length == 9
    assert np.array_equal(a.state_save(), b.state_save())
    assert np.array_equal(a.step_argmax([3]), b.step_argmax([3]))
    # a second rollback of the same snapshot is refused (more than one step ran)
    import qwisp_b200 as Q
    with pytest.raises(Q.SeedlessError):
        a.rollback(snap)
    a.close(); b.close()


def test_rollback_refused_unless_exactly_one_call_ran(tiny_engine):
    """The snapshot undoes ONE call.  After two or three calls the other ping-pong side no longer holds
    the snapshot's state (after three the parity alone would look right): the rollback is refused."""
    import qwisp_b200 as Q
    V = TINY["vocab"]
    a = tiny_engine.stream(64)
    a.step_argmax(prompt(V, 5, "rb3"))
    for ncalls in (2, 3):
        snap = a.snapshot()
        for i in range(ncalls):
            a.step_argmax([i + 1])
        with pytest.raises(Q.SeedlessError) as ei:
            a.rollback(snap)
        assert ei.value.code == -1
    snap = a.snapshot()
    a.chained_step_argmax(3, 3)                 # three chained steps are three calls
    with pytest.raises(Q.SeedlessError):
        a.rollback(snap)
    snap = a.snapshot()
    n = a.length
    a.step_argmax([4, 5, 6])                    # one call of three rows: allowed
    a.rollback(snap)
    assert a.length == n
    a.close()


def test_full_snapshot_restore(tiny_engine):
    V = TINY["vocab"]
    p = prompt(V, 6, "full")
    a = tiny_engine.stream(64)
    a.step_argmax(p)
    snap = a.full_snapshot()
    ref_blob = a.state_save()
    t1 = a.step_argmax([1, 2, 3])
    a.step_argmax([4])
    a.full_restore(snap)
    assert a.length == 6
    assert np.array_equal(a.state_save(), ref_blob)
    assert np.array_equal(a.step_argmax([1, 2, 3]), t1)
    a.close()


def test_state_blob_cross_arena_and_oracle_interop(tiny_engine, tiny_oracle):
    """lane_admit_restore_cross_arena_bitexact + blob interop with the oracle's writer."""
    V = TINY["vocab"]
    p = prompt(V, 9, "blob")
    a = tiny_engine.stream(48)
    a.step_argmax(p)
    blob = a.state_save()
    b = tiny_engine.stream(96)                  # different arena size
    assert b.state_restore(blob)
    nxt = [7, 11, 13]
    assert np.array_equal(a.step_argmax(nxt), b.step_argmax(nxt))
    c = tiny_engine.stream(48)
    assert not c.state_restore(blob[:-2])       # truncated
    bad = blob.copy(); bad[0] ^= 0xFF
    assert not c.state_restore(bad)
    small = tiny_engine.stream(4)
    assert not small.state_restore(blob)
    # the oracle can read a GPU blob and continues with near-identical logits
    so = tiny_oracle.stream(64)
    assert so.state_restore(blob)
    d = tiny_engine.stream(64); assert d.state_restore(blob)
    _, rl = so.step([5], want_logits=True)
    gl = d.step_logits([5])
    assert f16_report(gl, rl)["max_abs"] <= 2e-2
    for s in (a, b, c, small, d):
        s.close()


def test_lane_batch_equals_solo(tiny_engine):
    """lane_batch_argmax_bitexact: B=3 lanes with different histories == each lane solo, 4 steps."""
    V = TINY["vocab"]
    lens = [3, 8, 5]
    solo, lane = [], []
    for i, n in enumerate(lens):
        p = prompt(V, n, f"lane{i}")
        s1, s2 = tiny_engine.stream(64), tiny_engine.stream(64)
        f1, f2 = int(s1.step_argmax(p)[-1]), int(s2.step_argmax(p)[-1])
        assert f1 == f2
        solo.append((s1, f1)); lane.append((s2, f2))
    cur_solo = [f for _, f in solo]
    cur_lane = [f for _, f in lane]
    for _ in range(4):
        cur_solo = [int(s.step_argmax([t])[0]) for (s, _), t in zip(solo, cur_solo)]
        cur_lane = [int(t) for t in tiny_engine.batch_step_argmax([s for s, _ in lane], cur_lane)]
        assert cur_solo == cur_lane
    for (s1, _), (s2, _) in zip(solo, lane):
        assert np.array_equal(s1.state_save(), s2.state_save())
        s1.close(); s2.close()


def test_lane_batch_slots_protocol(tiny_engine):
    """BatchSlots: resumable chunked prefill with forward progress, batched step, release."""
    import qwisp_b200 as Q
    V = TINY["vocab"]
    slots = Q.LaneBatchSlots(tiny_engine, slot_count=3, chunk=4, default_seq_budget=64)
    p0, p1 = list(prompt(V, 10, "slot0")), list(prompt(V, 3, "slot1"))
    r = slots.admit_step(p0, 0, token_budget=1)           # budget below one chunk: still one whole chunk
    assert r == ("prefilling", 4)
    r = slots.admit_step(p0, 0, token_budget=8)
    assert r[0] == "done" and r[2] == 6
    first0 = r[1]
    first1 = slots.admit(p1, 1)
    ref = tiny_engine.stream(64)
    assert int(ref.step_argmax(p0)[-1]) == first0
    out = slots.step([first0, first1, None])
    assert out[2] is None and out[0] == int(ref.step_argmax([first0])[0])
    slots.release(0); slots.release(1)
    ref.close()


def test_sizes_and_errors(tiny_engine):
    import qwisp_b200 as Q
    s = tiny_engine.stream(8)
    with pytest.raises(Q.SeedlessError) as ei:
        s.step_argmax(list(range(9)))                   # beyond max_seq_len
    assert ei.value.code == -5
    with pytest.raises(Q.SeedlessError) as ei:
        s.step_argmax([TINY["vocab"]])                  # token id out of range
    assert ei.value.code == -1
    with pytest.raises(Q.SeedlessError) as ei:
        s.step_argmax(list(range(65)))                  # rows > max_rows
    assert ei.value.code == -5
    assert s.length == 0
    s.step_argmax([1, 2, 3])
    assert s.length == 3
    s.reset()
    assert s.length == 0
    s.close()


def test_fault_firewall():
    """gpu-failure-firewall: an injected failure poisons that engine only, stickily."""
    import qwisp_b200 as Q
    e1, e2 = gpu_engine(TINY, max_streams=2), gpu_engine(TINY, max_streams=2)
    try:
        s1, s2 = e1.stream(16), e2.stream(16)
        assert e1.gpu_fault() is None
        e1.inject_fault()
        bk = Q.SpecBackend(s1)
        assert bk.step_argmax([1]) is None
        assert "injected" in bk.gpu_fault()
        assert bk.step_argmax([1]) is None and bk.forward([1]) is None      # sticky
        with pytest.raises(Q.SeedlessError) as ei:
            s1.step_argmax([1])
        assert ei.value.code == -4
        assert e2.gpu_fault() is None
        assert len(s2.step_argmax([1, 2])) == 2                              # the other engine is unaffected
    finally:
        e1.close(); e2.close()


def test_device_wait_timeout_poisons_engine():
    """The device-side half of the firewall: a kernel whose bounded wait runs out (nothing arms the
    barrier; a thousand polls, no fault, no hang) leaves its code in the engine's error word, the call that
    synchronises next returns SL_ERR_CUDA, and the engine stays poisoned."""
    import qwisp_b200 as Q
    e = gpu_engine(TINY, max_streams=2)
    try:
        s = e.stream(16)
        assert len(s.step_argmax([1, 2])) == 2 and e.gpu_fault() is None
        e.debug_wait_timeout()
        with pytest.raises(Q.SeedlessError) as ei:
            s.step_argmax([3])
        assert ei.value.code == -3
        assert "bounded wait" in e.gpu_fault()
        with pytest.raises(Q.SeedlessError) as ei:
            s.step_argmax([3])
        assert ei.value.code == -4                                          # sticky
        assert Q.SpecBackend(s).forward([1]) is None
    finally:
        e.close()


def test_draft_tokens_out_of_range_are_refused(mini_engine):
    """A draft id is an index into the logits row on the device: anything outside [-1, vocab) is refused
    on the host, before a launch, and the stream does not advance."""
    import qwisp_b200 as Q
    V = MINI["vocab"]
    s = mini_engine.stream(16)
    for bad in (V, V + 5, -2):
        with pytest.raises(Q.SeedlessError) as ei:
            s.step_sample_rows([1, 2], [3, bad], 1.0, 1.0, 1, 2, 0)
        assert ei.value.code == -1
        assert s.length == 0
    logits = np.zeros((2, V), np.float16)
    with pytest.raises(Q.SeedlessError) as ei:
        Q.ops.sample_rows(mini_engine, logits, np.array([0, V], np.int32), 1.0, 1.0, 1, 2, 0)
    assert ei.value.code == -1
    assert mini_engine.gpu_fault() is None
    full, _, _ = s.step_sample_rows([1, 2], [3, V - 1], 0.0, 1.0, 1, 2, 0)
    assert len(full) == 2
    s.close()


def test_prefill_mode_vs_oracle_and_chunk_split_invariance(mini_oracle):
    """The prefill-only forward (dense projections on the tcgen05 GEMM) on 256 rows: within tolerance of
    the oracle, deterministic, and bit-identical however the prompt is cut into calls -- 256 = 128 + 128
    = 100 + 156 = 4 x 64 = 250 + 6 = 1 + 254 + 1 = 7 + 9 + 33 + 207 (the reference locks the same for its prefill kernel,
    SeedlessVerifyTests.swift:5811-5845).  Which family runs is a property of the entry point: the strict
    forward gives the same bits for 256 rows in one call as in 32-row calls."""
    V = MINI["vocab"]
    eng = gpu_engine(MINI, max_rows=256, max_streams=8, kv_pages=64)
    try:
        toks = prompt(V, 256, "hybrid")
        ref = mini_oracle.stream(320).forward(toks)
        outs = {}
        for name, cuts in (("256", [256]), ("128+128", [128, 128]), ("100+156", [100, 156]), ("4x64", [64] * 4), ("250+6", [250, 6]),
                           ("1+254+1", [1, 254, 1]), ("7+9+33+207", [7, 9, 33, 207])):
            s = eng.stream(320)
            pos, parts = 0, []
            for m in cuts:
                parts.append(s.forward_hybrid(toks[pos:pos + m])); pos += m
            outs[name] = (np.concatenate(parts), s.state_save())
            s.close()
        rep = f16_report(outs["256"][0], ref)
        print("prefill mode vs oracle", rep)
        assert np.isfinite(outs["256"][0].astype(np.float32)).all()
        # two free-running layers over 256 rows hold 512 routing decisions; a near-tie that falls the other way
        # on a row moves that row's hidden state visibly, so the bound is on the bulk, with a loose cap on outliers
        d256 = np.abs(outs["256"][0].astype(np.float32) - ref.astype(np.float32))
        rows_off = float((d256.max(axis=1) > 5e-2).mean())
        print("prefill mode: rows beyond 5e-2:", rows_off, "element quantile 0.99:", float(np.quantile(d256, 0.99)))
        assert rep["mean_abs"] <= 5e-3 and float(np.quantile(d256, 0.99)) <= 2e-2 and rows_off <= 0.05 and rep["max_abs"] <= 0.5, rep
        for name, (h, blob) in outs.items():
            assert np.array_equal(h.view(np.uint16), outs["256"][0].view(np.uint16)), name
            assert np.array_equal(blob, outs["256"][1]), name
        # strict mode: one 256-row call == eight 32-row calls, bit for bit, and close to the oracle
        a, b = eng.stream(320), eng.stream(320)
        ha = a.forward(toks)
        hb = np.concatenate([b.forward(toks[i:i + 32]) for i in range(0, 256, 32)])
        assert np.array_equal(ha.view(np.uint16), hb.view(np.uint16))
        assert np.array_equal(a.state_save(), b.state_save())
        rep_s = f16_report(ha, ref)
        print("strict 256 rows vs oracle", rep_s)
        ds = np.abs(ha.astype(np.float32) - ref.astype(np.float32))
        assert rep_s["mean_abs"] <= 5e-3 and float(np.quantile(ds, 0.99)) <= 2e-2 and float((ds.max(axis=1) > 5e-2).mean()) <= 0.05 and rep_s["max_abs"] <= 0.5, rep_s
        ta = a.step_argmax([5]); tb = b.step_argmax([5])
        assert np.array_equal(ta, tb)
        # the Tell closure set sees the library's own chunk size
        import qwisp_b200 as Q
        assert Q.SpecBackend(a).hybrid_chunk == 256
        a.close(); b.close()
    finally:
        eng.close()


def test_engine_from_host_tensors(tiny_oracle):
    """The weight-loading boundary: tensors handed over by name in the MLX layout."""
    import qwisp_b200 as Q
    from conftest import JITTER, CONV_STD
    cfg = Q.config(**TINY, max_rows=16, max_streams=2, kv_page_size=32, kv_pages=8)
    tensors = {n: tiny_oracle.tensor_bytes(n).copy() for n in tiny_oracle.tensor_names()}
    eng = Q.Engine.from_tensors(cfg, tensors)
    ref = gpu_engine(TINY, max_rows=16, max_streams=2, kv_pages=8)
    try:
        p = prompt(TINY["vocab"], 7, "host")
        a, b = eng.stream(32), ref.stream(32)
        assert np.array_equal(a.step_logits(p).view(np.uint16), b.step_logits(p).view(np.uint16))
        missing = dict(tensors); missing.pop("embed")
        with pytest.raises(Q.SeedlessError):
            Q.Engine.from_tensors(cfg, missing)
    finally:
        eng.close(); ref.close()


def test_engine_accepts_q4_embedding(tiny_oracle):
    """The checkpoint's 4-bit embedding table handed over as embed.w/.s/.b: the table the engine
    holds equals the reference's per-row dequantisation (embed_rows_q4,
    SeedlessFusedVerify.swift:556-570) bit for bit, and a step over it equals a step of an engine
    that was given those fp16 rows directly."""
    import qwisp_b200 as Q
    from oracle import oracle as O
    cfg = Q.config(**TINY, max_rows=16, max_streams=2, kv_page_size=32, kv_pages=8)
    V, H = TINY["vocab"], TINY["hidden"]
    w, s, b = O.synth_q4(SEED, "embed.q4", V, H)
    want = O.dequant_q4_half(w, s, b)
    tensors = {n: tiny_oracle.tensor_bytes(n).copy() for n in tiny_oracle.tensor_names()}
    q4 = dict(tensors); q4.pop("embed"); q4.update({"embed.w": w, "embed.s": s, "embed.b": b})
    f16 = dict(tensors); f16["embed"] = want
    a, bb = Q.Engine.from_tensors(cfg, q4), Q.Engine.from_tensors(cfg, f16)
    try:
        got = a.read_tensor("embed").view(np.uint16).reshape(V, H)
        assert np.array_equal(got, want.view(np.uint16))
        p = prompt(V, 7, "q4embed")
        assert np.array_equal(a.stream(32).step_logits(p).view(np.uint16), bb.stream(32).step_logits(p).view(np.uint16))
        both = dict(q4); both["embed"] = want
        with pytest.raises(Q.SeedlessError):
            Q.Engine.from_tensors(cfg, both)
        short = dict(q4); short["embed.s"] = s[:-1]
        with pytest.raises(Q.SeedlessError):
            Q.Engine.from_tensors(cfg, short)
    finally:
        a.close(); bb.close()


def test_engine_accepts_q8_router_and_shared_gate(tiny_oracle):
    """The checkpoint's 8-bit group-64 router / shared gate handed over as L<i>.moe.router.w/.s/.b and
    L<i>.moe.shared_gate.w/.s/.b (qmm8, SeedlessMetalForward.swift:384-434): routing indices bit-exact
    against the CPU restatement with the same 8-bit tensors, MoE output and model logits within tolerance."""
    import qwisp_b200 as Q
    from oracle import oracle as O
    from conftest import oracle_model
    cfg = Q.config(**TINY, max_rows=16, max_streams=2, kv_page_size=32, kv_pages=8)
    H, E, nl = TINY["hidden"], TINY["n_experts"], TINY["n_layers"]
    tensors = {n: tiny_oracle.tensor_bytes(n).copy() for n in tiny_oracle.tensor_names()}
    ref = oracle_model(TINY)                     # own copy: the shared fixture keeps its fp16 router
    for i in range(nl):
        r16 = tensors.pop(f"L{i}.moe.router").view(np.float16).reshape(E, H)
        g16 = tensors.pop(f"L{i}.moe.shared_gate").view(np.float16).reshape(1, H)
        rw, rs, rb = O.quantize_q8(r16)
        gw, gs, gb = O.quantize_q8(g16)
        tensors.update({f"L{i}.moe.router.w": rw, f"L{i}.moe.router.s": rs, f"L{i}.moe.router.b": rb,
                        f"L{i}.moe.shared_gate.w": gw, f"L{i}.moe.shared_gate.s": gs, f"L{i}.moe.shared_gate.b": gb})
        ref.set_router_q8(i, rw, rs, rb, gw, gs, gb)
    eng = Q.Engine.from_tensors(cfg, tensors)
    try:
        for T in (1, 9):
            x = O.synth_f16(SEED, f"q8router.x{T}", T * H, 0.0, 1.0).reshape(T, H)
            for layer in (0, nl - 1):
                out, inds, scores = Q.ops.moe_block(eng, layer, x)
                ro, ri, rs_ = ref.moe_block(layer, x)
                assert np.array_equal(inds, ri), ("routing indices differ", T, layer)
                assert f16_report(scores, rs_)["max_abs"] <= 2e-3
                assert f16_report(out, ro)["max_abs"] <= 2e-2
        p = prompt(TINY["vocab"], 7, "q8router")
        lg = eng.stream(32).step_logits(p)
        _, rl = ref.stream(32).step(p, want_logits=True)
        rep = f16_report(lg, rl)
        print("q8 router model logits", rep)
        assert rep["max_abs"] <= 2e-2, rep
        part = dict(tensors); part.pop("L0.moe.shared_gate.b")
        with pytest.raises(Q.SeedlessError):
            Q.Engine.from_tensors(cfg, part)
    finally:
        eng.close(); ref.close()


def test_engine_f32_gdn_norm_weight(tiny_oracle):
    """A GDN norm weight handed over as f32 ("L<i>.gdn.norm.f32"): the gated norm keeps its normed value in
    f32 (the reference's promoted variant, SeedlessFusedVerify.swift:766-813, 2815-2818).  Weights that fp16
    cannot hold make the two variants differ; the GDN layer output is compared with the CPU restatement
    given the same f32 weight."""
    import qwisp_b200 as Q
    from oracle import oracle as O
    from conftest import oracle_model
    cfg = Q.config(**TINY, max_rows=16, max_streams=4, kv_page_size=32, kv_pages=8)
    H, nl = TINY["hidden"], TINY["n_layers"]
    tensors = {n: tiny_oracle.tensor_bytes(n).copy() for n in tiny_oracle.tensor_names()}
    ref = oracle_model(TINY)
    gdn_layers = [i for i in range(nl) if (i + 1) % TINY["attn_every"] != 0]
    for i in gdn_layers:
        w16 = tensors.pop(f"L{i}.gdn.norm").view(np.float16)
        w32 = (w16.astype(np.float32) * np.float32(1.0003) + np.float32(1e-4) * np.sin(np.arange(128, dtype=np.float32))).astype(np.float32)
        assert not np.array_equal(w32.astype(np.float16).astype(np.float32), w32)
        tensors[f"L{i}.gdn.norm.f32"] = w32
        ref.set_gdn_norm_f32(i, w32)
    eng = Q.Engine.from_tensors(cfg, tensors)
    plain = gpu_engine(TINY, max_rows=16, max_streams=4, kv_pages=8)
    try:
        layer = gdn_layers[0]
        x = O.synth_f16(SEED, "f32norm.x", 5 * H, 0.0, 1.0).reshape(5, H)
        want = ref.stream(32).mixer_rows(layer, x, 0)
        got = Q.ops.mixer(eng.stream(32), layer, x, 0)
        rep = f16_report(got, want)
        print("f32 gdn norm", rep)
        assert rep["max_abs"] <= 2e-2, rep
        assert rep["max_abs"] <= 1e-3, rep                          # fp16 rounding of the out-projection apart
        other = Q.ops.mixer(plain.stream(32), layer, x, 0)          # fp16 weight variant: measurably different
        assert not np.array_equal(other.view(np.uint16), got.view(np.uint16))
        p = prompt(TINY["vocab"], 7, "f32norm")
        lg = eng.stream(32).step_logits(p)
        _, rl = ref.stream(32).step(p, want_logits=True)
        assert f16_report(lg, rl)["max_abs"] <= 2e-2
        bad = dict(tensors); bad[f"L{layer}.gdn.norm.f32"] = np.zeros(64, np.float32)
        with pytest.raises(Q.SeedlessError):
            Q.Engine.from_tensors(cfg, bad)
    finally:
        eng.close(); plain.close(); ref.close()


def test_step_sample_rows_greedy_equals_argmax(mini_engine):
    """At temperature 0 the sampling step returns the argmax step's tokens (stepSampleRows with
    invT <= 0, SamplerGPU.swift:13-15) and leaves the caches in the same state."""
    import qwisp_b200 as Q
    prompt = Q.ops.synth_tokens(SEED, "sample.prompt", 9, mini_engine.cfg.vocab)
    a, b = mini_engine.stream(64), mini_engine.stream(64)
    ta = a.step_argmax(prompt)
    full, resid, acc = b.step_sample_rows(prompt, None, 0.0, 1.0, 1, 2, 0)
    assert np.array_equal(ta, full) and np.array_equal(full, resid) and not acc.any()
    nxt_a = a.step_argmax([int(ta[-1])])
    nxt_b, _, _ = b.step_sample_rows([int(full[-1])], [int(nxt_a[0])], 0.0, 1.0, 1, 2, 9)
    assert np.array_equal(nxt_a, nxt_b)
    a.close(); b.close()


def test_speculative_loop_equals_greedy_on_gpu(tiny_engine):
    """Tell-style greedy speculation (suffix draft, multi-row verify, rollback + replay) over the
    CUDA backend returns exactly the plain greedy stream."""
    from qwisp_b200.engine import SpecBackend
    from qwisp_b200.tell import SpecStats, speculative_greedy
    prompt = [7, 8, 9, 10, 7, 8, 9, 10, 7, 8, 9]
    n_new = 40
    s0 = tiny_engine.stream(256)
    out = s0.step_argmax(prompt)
    want = [int(out[-1])]
    while len(want) < n_new:
        want.append(int(s0.step_argmax([want[-1]])[0]))
    s1 = tiny_engine.stream(256)
    stats = SpecStats()
    got = speculative_greedy(SpecBackend(s1, hybrid_chunk=8), prompt, n_new, chunk=8, min_match=1, stats=stats)
    assert got == want, (got, want)
    # the verify / reject / rollback / replay sequence, driven by hand with a right and a wrong draft
    s2 = tiny_engine.stream(256)
    bk = SpecBackend(s2, hybrid_chunk=8)
    first = bk.step_argmax(prompt)[-1]
    assert first == want[0]
    out = bk.step_argmax([want[0], want[1], want[2]])            # a draft that is right: every row confirms the next
    assert out == want[1:4]
    snap = bk.snapshot()
    wrong = (want[4] + 1) % tiny_engine.cfg.vocab
    out = bk.step_argmax([want[3], wrong, want[5]])              # second row is a wrong draft
    assert out[0] == want[4]
    bk.rollback(snap)
    redo = bk.step_argmax([want[3]])
    assert redo == [want[4]]
    cont = [want[4]]
    while len(cont) < 8:
        cont.append(bk.step_argmax([cont[-1]])[0])
    assert cont == want[4:12]
    s0.close(); s1.close(); s2.close()
