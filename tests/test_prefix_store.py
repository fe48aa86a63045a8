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
        slots = Q.LaneBatchSlots(eng, 2, chunk=8, default_seq_budget=64, prefix_store=store)
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
