"""RAM prefix store semantics (PrefixPersist.swift:196-235) and its use at admission."""
import numpy as np
import pytest

from qwisp_b200.prefix import PrefixRAMStore


def test_store_longest_prefix_supersede_and_lru():
    st = PrefixRAMStore(budget=100)
    st.save([1, 2, 3], b"a" * 30)
    st.save([9, 9], b"b" * 30)
    assert st.best_match([1, 2]) is None                       # only whole-key prefixes match
    assert st.best_match([1, 2, 3, 4])[0] == (1, 2, 3)
    st.save([1, 2, 3, 4, 5], b"c" * 30)                        # supersedes its own prefix [1,2,3]
    assert [k for k, _ in st.entries] == [(1, 2, 3, 4, 5), (9, 9)]
    assert st.best_match([1, 2, 3, 4, 5, 6])[1] == b"c" * 30
    st.save([7], b"d" * 30)
    st.save([8], b"e" * 30)                                    # 120 bytes > 100: the least recently used goes
    assert st.nbytes <= 100 and (9, 9) not in [k for k, _ in st.entries]
    assert st.best_match([9, 9, 1]) is None
    hit = st.best_match([1, 2, 3, 4, 5])                       # a match moves the entry to the front
    assert hit is not None and st.entries[0][0] == (1, 2, 3, 4, 5)
    st.save([5], b"x" * 101)                                   # larger than the whole budget: ignored
    assert (5,) not in [k for k, _ in st.entries]
    off = PrefixRAMStore(0)
    off.save([1], b"zz")
    assert off.entries == [] and off.best_match([1]) is None
    st.remove_all()
    assert st.entries == []


def test_max_common_prefix_is_a_partial_match():
    st = PrefixRAMStore(budget=1000)
    st.save([1, 2, 3, 4], b"a")
    st.save([9, 8, 7], b"b")
    order = [k for k, _ in st.entries]
    assert st.max_common_prefix([1, 2, 3, 9, 9]) == 3
    assert st.max_common_prefix([1, 2, 3, 4, 5, 6]) == 4
    assert st.max_common_prefix([9, 1]) == 1 and st.max_common_prefix([5]) == 0 and st.max_common_prefix([]) == 0
    assert [k for k, _ in st.entries] == order                 # no MRU side effect
    assert PrefixRAMStore(0).max_common_prefix([1, 2]) == 0


def test_admit_plan_boundaries():
    """The reference's own self-check of the admission plan (LaneServe.swift:133-156), case by case."""
    from qwisp_b200.engine import LaneAdmitPlan, admit_plan
    p = lambda n, hit, lcp: admit_plan(n, hit, lcp, 1024)
    assert p(9000, 0, 0) == LaneAdmitPlan(0, None, True)                   # cold first request
    assert p(12000, 0, 9000) == LaneAdmitPlan(0, 9000, True)               # second same-prefix request: capture at the exact boundary
    assert p(12000, 9000, 9000) == LaneAdmitPlan(9000, None, True)         # third: warm restore, no re-capture
    assert p(4000, 0, 900) == LaneAdmitPlan(0, None, True)                 # shared prefix below min_shared
    assert p(12000, 8900, 9000) == LaneAdmitPlan(8900, None, True)         # capture not worth a blob copy
    assert p(9000, 0, 9000) == LaneAdmitPlan(0, 8999, True)                # lcp clamps to prompt_len - 1
    assert p(800, 0, 0) == LaneAdmitPlan(0, None, False)                   # short prompt: not cached
    assert p(9000, 8999, 8999) == LaneAdmitPlan(8999, None, False)         # restore covers everything but the last token


@pytest.mark.gpu
def test_shared_prefix_is_captured_at_the_exact_boundary_and_reused():
    """Three prompts that share their first 300 tokens: the first is served cold and leaves its prompt-end state; the
    second sees the partial match, splits a chunk at token 300 and captures the state there; the third restores
    those 300 tokens and prefills only its tail.  Tokens of all three equal cold lone streams (prefill mode)."""
    import qwisp_b200 as Q
    from conftest import SEED, TINY, gpu_engine
    from oracle import oracle as O
    eng = gpu_engine(TINY, max_rows=32, max_streams=8, kv_pages=64)
    try:
        shared, conv = Q.PrefixRAMStore(budget=64 << 20), Q.PrefixRAMStore(budget=64 << 20)
        slots = Q.LaneBatchSlots(eng, 3, chunk=16, default_seq_budget=128, prefix_store=conv, shared_store=shared, hybrid=True, min_shared=32)
        # (a capture must beat the restore point by 256 tokens, so the common part is 300 tokens long)
        common = [int(t) for t in O.synth_tokens(SEED, "shared.common", 300, TINY["vocab"])]
        tails = [[int(t) for t in O.synth_tokens(SEED, f"shared.tail{i}", 9 + 4 * i, TINY["vocab"])] for i in range(3)]
        prompts = [common + t for t in tails]
        eng2 = gpu_engine(TINY, max_rows=32, max_streams=8, kv_pages=64)
        firsts = []
        for i, pr in enumerate(prompts):
            r = slots.admit_step(pr, i, 1 << 20, 400)
            assert r[0] == "done"
            firsts.append(r[1])
        assert slots.captures == 1 and slots.restore_hits == 1 and slots.restored_tokens == 300
        assert [len(k) for k, _ in shared.entries] == [300]
        got = [[f] for f in firsts]
        cur = list(firsts)
        for _ in range(3):
            cur = slots.step(cur)
            for i in range(3):
                got[i].append(cur[i])
        for i, pr in enumerate(prompts):
            lone = eng2.stream(400)
            pos, normed = 0, None
            while pos < len(pr):
                n = min(16, len(pr) - pos)
                normed = lone.forward_hybrid(pr[pos:pos + n]); pos += n
            want = [int(Q.ops.lm_head(eng2, normed[-1:], want_logits=False)[1][0])]
            for _ in range(3):
                want.append(int(lone.step_argmax([want[-1]])[0]))
            lone.close()
            assert got[i] == want, i
        eng2.close()
    finally:
        eng.close()


@pytest.mark.gpu
def test_admission_restores_the_longest_stored_prefix():
    """A second request that extends a served prompt starts from the stored state: only the suffix is
    prefilled and charged, and its tokens equal those of a cold lone stream."""
    import qwisp_b200 as Q
    from conftest import SEED, TINY, gpu_engine
    from oracle import oracle as O
    eng = gpu_engine(TINY, max_rows=32, max_streams=8, kv_pages=64)
    try:
        store = Q.PrefixRAMStore(budget=64 << 20)
        slots = Q.LaneBatchSlots(eng, 2, chunk=8, default_seq_budget=64, prefix_store=store, min_shared=8)
        base = [int(t) for t in O.synth_tokens(SEED, "prefix.base", 20, TINY["vocab"])]
        ext = base + [int(t) for t in O.synth_tokens(SEED, "prefix.ext", 7, TINY["vocab"])]
        r1 = slots.admit_step(base, 0, 1 << 20, 64)
        assert r1[0] == "done" and r1[2] == 20 and slots.restored_tokens == 0
        slots.release(0)
        r2 = slots.admit_step(ext, 1, 1 << 20, 64)
        assert r2[0] == "done" and slots.restored_tokens == 20 and r2[2] == 7
        got = [r2[1]]
        for _ in range(4):
            got.append(slots.step([None, got[-1]])[1])
        slots.release(1)
        lone = eng.stream(64)
        want = [int(lone.step_argmax(ext)[-1])]
        for _ in range(4):
            want.append(int(lone.step_argmax([want[-1]])[0]))
        lone.close()
        assert got == want
        assert [len(k) for k, _ in store.entries] == [27]       # the longer conversation superseded its prefix
    finally:
        eng.close()


def test_qwp1_layout_and_disk_store(tmp_path):
    """The disk tier's file layout and policy, following the reference's own self-check
    (PrefixPersist.swift:162-215): round trip, longest prefix, model isolation, LRU caps."""
    import os
    import struct
    import time
    from qwisp_b200.prefix import PrefixDiskStore, fnv1a64, qwp1_decode, qwp1_encode
    state = bytes(range(64))
    blob = qwp1_encode("/m", [1, 2, 3], state)
    assert blob[:4] == b"QWP1" and struct.unpack_from("<II", blob, 4) == (1, 2)
    assert blob[12:14] == b"/m" and struct.unpack_from("<I", blob, 14)[0] == 3
    assert struct.unpack_from("<3i", blob, 18) == (1, 2, 3) and blob[30:] == state
    assert qwp1_decode(blob) == ("/m", [1, 2, 3], state)
    assert qwp1_decode(blob[:20]) is None and qwp1_decode(b"XXXX" + blob[4:]) is None
    assert fnv1a64(b"") == 0xCBF29CE484222325 and fnv1a64(b"a") == 0xAF63DC4C8601EC8C
    d = str(tmp_path / "prefix")
    st = PrefixDiskStore(d, "/m", max_slots=4)
    a, ab = [1, 2, 3, 4], [1, 2, 3, 4, 5, 6]
    st.save(a, state); st.save(ab, state + state)
    PrefixDiskStore(d, "/other").save(ab + [7], state)
    assert st.best_match(ab + [9, 9]) == (ab, state + state)
    assert st.best_match([1, 2, 3, 4, 99]) == (a, state)
    assert PrefixDiskStore(d, "/nope").best_match(ab) is None
    assert st.best_match([8, 8, 8]) is None
    assert st.has(a) and not st.has([77, 78]) and st.restore_hits == 2
    with open(os.path.join(d, "prefix-garbage.bin"), "wb") as f:
        f.write(b"not a prefix file")
    assert st.best_match(ab) == (ab, state + state)             # a malformed file is skipped
    os.remove(os.path.join(d, "prefix-garbage.bin"))
    for i in range(6):
        st.save([100, i], state)
        time.sleep(0.002)
    assert len([n for n in os.listdir(d) if n.endswith(".bin")]) == 4
    assert st.has([100, 5]) and not st.has(a)                   # the oldest went first
    one = max(os.path.getsize(os.path.join(d, n)) for n in os.listdir(d))
    st.evict(budget=one)
    assert len([n for n in os.listdir(d) if n.endswith(".bin")]) == 1
    st.save([5], b"x" * 10); big = PrefixDiskStore(d, "/m", max_bytes=4)
    big.save([6], b"y" * 10)
    assert not big.has([6])                                     # above the per-entry cap: not written
