"""The lane admission path (`LaneBatchSlots`, after LaneServe.swift:331-485) on a scripted engine: where a prompt is
cut into calls, what is captured, restored and charged.  No GPU: the engine below only records calls and derives its
outputs from the token history, so a restored stream and a cold one can be compared exactly."""
import numpy as np

from qwisp_b200.engine import LaneBatchSlots
from qwisp_b200.prefix import PrefixRAMStore
from qwisp_b200.scheduler import ContinuousScheduler, Request


class _Cfg:
    kv_page_size, kv_pages, max_rows, hidden = 16, 4096, 64, 4


def _digest(history):
    h = 1469598103934665603
    for t in history:
        h = ((h ^ int(t)) * 1099511628211) % (1 << 61)
    return h


class FakeStream:
    def __init__(self, engine, max_seq_len):
        self.engine, self.max_seq_len, self.history, self.calls = engine, max_seq_len, [], []

    def _run(self, tokens, kind):
        self.calls.append((kind, len(tokens)))
        self.history.extend(int(t) for t in tokens)
        assert len(self.history) <= self.max_seq_len

    def forward_hybrid(self, tokens, want_hidden=True):
        self._run(tokens, "hybrid")
        return np.full((len(tokens), _Cfg.hidden), float(_digest(self.history) % 1000), dtype=np.float32) if want_hidden else None

    def forward(self, tokens, want_hidden=True):
        self._run(tokens, "strict")

    def step_argmax(self, tokens):
        self._run(tokens, "step")
        return np.array([_digest(self.history) % 997] * len(tokens), dtype=np.int32)

    def state_save(self):
        return np.array(self.history, dtype=np.int64).tobytes() or b"\0"

    def state_restore(self, blob):
        self.history = [int(t) for t in np.frombuffer(blob, dtype=np.int64)]
        return True

    def close(self):
        self.engine.closed += 1


class FakeEngine:
    cfg = _Cfg

    def __init__(self):
        self.streams, self.closed = [], 0

    def stream(self, max_seq_len):
        s = FakeStream(self, max_seq_len)
        self.streams.append(s)
        return s

    def lm_head_argmax(self, normed_rows):
        return np.array([int(normed_rows[-1][0]) % 997], dtype=np.int32)

    def batch_step_argmax(self, streams, tokens):
        return np.array([int(s.step_argmax([t])[0]) for s, t in zip(streams, tokens)], dtype=np.int32)


def _prompts():
    rng = np.random.RandomState(7)
    common = [int(t) for t in rng.randint(0, 5000, 300)]
    return common, [common + [int(t) for t in rng.randint(0, 5000, n)] for n in (9, 13, 40)]


def test_capture_at_the_exact_boundary_then_restore_and_charge_only_the_tail():
    eng = FakeEngine()
    shared, conv = PrefixRAMStore(1 << 20), PrefixRAMStore(1 << 20)
    slots = LaneBatchSlots(eng, 3, chunk=64, default_seq_budget=512, prefix_store=conv, shared_store=shared, hybrid=True, min_shared=32)
    common, prompts = _prompts()
    # first request: cold, whole chunks of 64, prompt-end state saved (it is the evidence of the recurrence)
    r0 = slots.admit_step(prompts[0], 0, 1 << 20, 512)
    assert r0[0] == "done" and r0[2] == 309
    assert [n for _, n in eng.streams[0].calls] == [64, 64, 64, 64, 53]
    assert slots.captures == 0 and [len(k) for k, _ in conv.entries] == [309] and shared.entries == []
    # second request: no whole-entry hit, partial match of 300 -> one chunk is cut at token 300 and the state captured there
    r1 = slots.admit_step(prompts[1], 1, 1 << 20, 512)
    assert r1[0] == "done" and r1[2] == 313
    assert [n for _, n in eng.streams[1].calls] == [64, 64, 64, 64, 44, 13]
    assert slots.captures == 1 and [len(k) for k, _ in shared.entries] == [300] and slots.restore_hits == 0
    # third request: restores the 300 tokens, prefills and is charged for its 40-token tail only, captures nothing new
    r2 = slots.admit_step(prompts[2], 2, 1 << 20, 512)
    assert r2[0] == "done" and r2[2] == 40
    assert [n for _, n in eng.streams[2].calls] == [40]
    assert slots.captures == 1 and slots.restore_hits == 1 and slots.restored_tokens == 300 and slots.prefilled_tokens == 309 + 313 + 40
    # a restored stream is in the state of a cold one: same first token, same decode
    cold = FakeEngine()
    cs = LaneBatchSlots(cold, 1, chunk=64, default_seq_budget=512, hybrid=True)
    want = cs.admit_step(prompts[2], 0, 1 << 20, 512)
    assert want[1] == r2[1] and eng.streams[2].history == cold.streams[0].history
    assert slots.step([None, None, r2[1]])[2] == cs.step([want[1]])[0]


def test_budget_resumes_mid_prompt_and_always_makes_one_chunk_of_progress():
    eng = FakeEngine()
    slots = LaneBatchSlots(eng, 1, chunk=64, default_seq_budget=512, hybrid=True)
    prompt = list(range(200))
    r = slots.admit_step(prompt, 0, token_budget=10, seq_budget=512)          # less than a chunk: one whole chunk runs anyway
    assert r == ("prefilling", 64)
    r = slots.admit_step(prompt, 0, token_budget=130, seq_budget=512)         # two more chunks fit, the third would not
    assert r == ("prefilling", 128)
    r = slots.admit_step(prompt, 0, token_budget=1, seq_budget=512)
    assert r[0] == "done" and r[2] == 8
    assert [n for _, n in eng.streams[0].calls] == [64, 64, 64, 8]
    slots.release(0)
    assert eng.closed == 1 and not slots.can_admit(10, 16 * 4096 + 1) and slots.can_admit(10, 512)


def test_strict_mode_prefills_with_forward_and_takes_the_first_token_from_the_last_chunk():
    eng = FakeEngine()
    slots = LaneBatchSlots(eng, 1, chunk=64, default_seq_budget=512, hybrid=False)
    r = slots.admit_step(list(range(100)), 0, 1 << 20, 512)
    assert r[0] == "done" and [k for k, _ in eng.streams[0].calls] == ["strict", "step"]


def test_scheduler_over_the_lane_slots_serves_a_shared_prefix_workload():
    """Eight requests, half of them with a common 300-token prefix, through the token-budget scheduler: everything finishes,
    the prefix is captured once and restored by the later sharers, and every stream's tokens equal a cold lone stream's."""
    eng = FakeEngine()
    shared, conv = PrefixRAMStore(1 << 22), PrefixRAMStore(1 << 22)
    slots = LaneBatchSlots(eng, 4, chunk=64, default_seq_budget=512, prefix_store=conv, shared_store=shared, hybrid=True, min_shared=32)
    sched = ContinuousScheduler(slots, token_budget=256)
    rng = np.random.RandomState(11)
    common = [int(t) for t in rng.randint(0, 5000, 300)]
    prompts = [(common if i % 2 == 0 else []) + [int(t) for t in rng.randint(0, 5000, 20 + 7 * i)] for i in range(8)]
    reqs = [sched.submit(Request(p, 5)) for p in prompts]
    sched.run_to_completion(max_rounds=400)
    assert all(r.finished and len(r.out) == 5 for r in reqs)
    assert slots.captures == 1 and slots.restore_hits >= 2 and slots.restored_tokens == 300 * slots.restore_hits
    for p, r in zip(prompts, reqs):
        lone = FakeEngine()
        ls = LaneBatchSlots(lone, 1, chunk=64, default_seq_budget=512, hybrid=True)
        first = ls.admit_step(p, 0, 1 << 20, 512)[1]
        want = [first]
        for _ in range(4):
            want.append(ls.step([want[-1]])[0])
        assert r.out == want
