"""Continuous-batching round policy (ContinuousBatch.swift:184-268) against a scripted engine, the way the
reference's own selfCheck tests it (ContinuousBatch.swift:270-330), and against single-stream decoding on the GPU."""
import numpy as np
import pytest

from qwisp_b200.scheduler import ContinuousScheduler, Request


class FakeSlots:
    """next token = last + 1; first token = prompt[0] + 1; prefill in chunks of `chunk` tokens."""

    def __init__(self, slot_count=2, chunk=4, capacity=10 ** 9):
        self.slot_count, self.chunk, self.capacity = slot_count, chunk, capacity
        self.pos = [None] * slot_count
        self.budget = [0] * slot_count
        self.max_busy = 0
        self.calls = []

    def _busy(self):
        self.max_busy = max(self.max_busy, sum(p is not None for p in self.pos))

    def can_admit(self, prompt_len, seq_budget):
        return sum(b for b, p in zip(self.budget, self.pos) if p is not None) + seq_budget <= self.capacity

    def admit_step(self, prompt, slot, token_budget, seq_budget=0):
        if prompt and prompt[0] < 0:
            return ("failed",)
        if self.pos[slot] is None:
            self.pos[slot] = 0; self.budget[slot] = seq_budget
        self._busy()
        consumed, first = 0, True
        while self.pos[slot] < len(prompt):
            n = min(self.chunk, len(prompt) - self.pos[slot])
            if not first and consumed + n > token_budget:
                break
            self.pos[slot] += n; consumed += n; first = False
        self.calls.append((slot, token_budget, consumed))
        if self.pos[slot] == len(prompt):
            return ("done", prompt[0] + 1, consumed)
        return ("prefilling", consumed)

    def step(self, last):
        self._busy()
        return [None if t is None else t + 1 for t in last]

    def release(self, slot):
        self.pos[slot] = None; self.budget[slot] = 0


def test_streams_complete_in_order_and_never_exceed_the_slots():
    fake = FakeSlots(slot_count=2)
    s = ContinuousScheduler(fake, token_budget=64)
    reqs = [s.submit(Request([100 * i], 4)) for i in range(5)]
    s.run_to_completion()
    for i, r in enumerate(reqs):
        assert r.finished and r.out == [100 * i + 1, 100 * i + 2, 100 * i + 3, 100 * i + 4]
    assert fake.max_busy <= 2 and s.max_running <= 2
    assert all(p is None for p in fake.pos)


def test_stop_token_is_not_emitted_and_max_tokens_caps():
    fake = FakeSlots()
    s = ContinuousScheduler(fake, token_budget=64)
    a = s.submit(Request([10], 10, frozenset({13})))       # 11, 12, then 13 stops
    b = s.submit(Request([20], 1))                          # a single token
    c = s.submit(Request([30], 0))                          # no-op
    d = s.submit(Request([40], 5, frozenset({41})))         # first token is a stop token
    e = s.submit(Request([-1], 5))                          # engine failure
    s.run_to_completion()
    assert a.out == [11, 12] and b.out == [21] and c.out == [] and d.out == [] and e.out == []
    assert all(r.finished for r in (a, b, c, d, e))


def test_budget_reserves_running_slots_and_charges_consumed_tokens():
    fake = FakeSlots(slot_count=2, chunk=4)
    s = ContinuousScheduler(fake, token_budget=9)
    long1 = s.submit(Request(list(range(1, 21)), 3))        # 20 prompt tokens
    long2 = s.submit(Request(list(range(50, 70)), 3))
    s.round()
    # first scheduling round: nothing running, pool 9: slot 0 consumes 8 (two chunks; a third would exceed), pool 1 left:
    # slot 1 still makes progress by one whole chunk (forward-progress guarantee)
    assert fake.calls[:2] == [(0, 9, 8), (1, 1, 4)]
    s.run_to_completion()
    assert long1.out == [2, 3, 4] and long2.out == [51, 52, 53]
    # once slot 0 runs, the pool shrinks by one for its decode step
    budgets_after_running = [tb for (slot, tb, _) in fake.calls if slot == 1]
    assert 8 in budgets_after_running or min(budgets_after_running) < 9


def test_head_of_line_gate_blocks_smaller_requests_behind_it():
    fake = FakeSlots(slot_count=2, capacity=40)
    s = ContinuousScheduler(fake, token_budget=64)
    big1 = s.submit(Request([1] * 20, 8))                   # needs 29
    s.round()                                               # big1 holds its arena from here on
    big2 = s.submit(Request([2] * 20, 4))                   # needs 25: must wait for big1
    small = s.submit(Request([3], 2))                       # would fit, but is behind big2
    s.round()
    assert len(s.queue) == 2 and s.queue[0] is big2          # small did not skip ahead
    s.run_to_completion()
    assert big1.out == list(range(2, 10)) and big2.out == [3, 4, 5, 6] and small.out == [4, 5]
    never = ContinuousScheduler(FakeSlots(capacity=5), token_budget=8)
    never.submit(Request([1] * 20, 4))
    with pytest.raises(RuntimeError):
        never.run_to_completion()


@pytest.mark.gpu
def test_scheduler_streams_equal_single_stream_decoding():
    """Five requests over three slots with a small token budget: every request's tokens equal the ones a
    lone stream produces for the same prompt (prefill chunking and batching leave rows bit-identical)."""
    import qwisp_b200 as Q
    from conftest import SEED, TINY, gpu_engine
    from oracle import oracle as O
    eng = gpu_engine(TINY, max_rows=32, max_streams=8, kv_pages=64)
    try:
        slots = Q.LaneBatchSlots(eng, 3, chunk=8, default_seq_budget=64)
        s = ContinuousScheduler(slots, token_budget=12)
        lens = [5, 19, 9, 30, 1]
        prompts = [[int(t) for t in O.synth_tokens(SEED, f"sched.p{i}", n, TINY["vocab"])] for i, n in enumerate(lens)]
        reqs = [s.submit(Request(p, 6)) for p in prompts]
        s.run_to_completion(max_rounds=500)
        assert s.max_running <= 3
        for p, r in zip(prompts, reqs):
            st = eng.stream(64)
            want = [int(st.step_argmax(p)[-1])]
            for _ in range(5):
                want.append(int(st.step_argmax([want[-1]])[0]))
            st.close()
            assert r.finished and r.out == want
    finally:
        eng.close()
