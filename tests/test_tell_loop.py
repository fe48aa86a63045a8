"""The speculation loop of qwisp_b200/tell.py on a CPU backend over the oracle: the speculative
token stream equals plain greedy decode, drafts get accepted on repetitive text, rejections roll
back.  (The same loop on the CUDA backend is in tests/test_gpu_engine.py.)"""
import numpy as np

from conftest import TINY, oracle_model


class OracleBackend:
    """step_argmax / snapshot / rollback over one oracle stream (whole-state snapshots)."""

    def __init__(self, model, max_seq_len=256):
        self.s = model.stream(max_seq_len)

    def step_argmax(self, tokens):
        return [int(t) for t in self.s.step(tokens)]

    def snapshot(self):
        return self.s.state_save()

    def rollback(self, snap):
        assert self.s.state_restore(snap)


def test_suffix_draft_rules():
    from qwisp_b200.tell import suffix_draft
    assert suffix_draft([1, 2, 3], min_match=2) == []                           # nothing repeats
    seq = [5, 6, 7, 8, 9, 5, 6, 7]
    assert suffix_draft(seq, max_match=8, draft_k=7, min_match=2, alpha=2) == [8, 9, 5, 6, 7]
    assert suffix_draft(seq, draft_k=2) == [8, 9]                               # capped by draft_k
    assert suffix_draft([1, 2, 9, 1, 2, 4, 1, 2], min_match=2, alpha=1) == [4, 1]   # tie between 9 and 4: most recent wins
    assert suffix_draft([1, 2, 9, 1, 2, 9, 1, 2, 4, 1, 2], min_match=2, alpha=1, max_match=2) == [9, 1]   # majority wins


def test_speculative_equals_greedy_on_oracle():
    from qwisp_b200.tell import SpecStats, speculative_greedy
    model = oracle_model(TINY)
    prompt = [7, 8, 9, 10, 7, 8, 9, 10, 7, 8, 9]
    n_new = 24
    plain = OracleBackend(model)
    out = plain.step_argmax(prompt)
    want = [out[-1]]
    while len(want) < n_new:
        want.append(plain.step_argmax([want[-1]])[0])
    stats = SpecStats()
    got = speculative_greedy(OracleBackend(model), prompt, n_new, chunk=4, stats=stats)
    assert got == want
    assert stats.rollbacks <= stats.verify_calls
    # a random-weight model rarely repeats itself; with single-token matches allowed the verify path runs too
    stats1 = SpecStats()
    got1 = speculative_greedy(OracleBackend(model), prompt, n_new, chunk=4, min_match=1, stats=stats1)
    assert got1 == want


class ToyBackend:
    """A deterministic next-token rule with a long period and occasional breaks in the pattern, so
    suffix drafts are mostly right and sometimes wrong.  Snapshot = sequence length."""

    def __init__(self):
        self.seq = []

    def _next(self):
        n = len(self.seq)
        a, b = self.seq[-1], (self.seq[-2] if n > 1 else 0)
        return (a + b * 2 + (1 if n % 11 == 0 else 0)) % 9

    def step_argmax(self, tokens):
        out = []
        for t in tokens:
            self.seq.append(int(t))
            out.append(self._next())
        return out

    def snapshot(self):
        return len(self.seq)

    def rollback(self, snap):
        del self.seq[snap:]


def test_speculation_accepts_and_rolls_back_on_toy_model():
    from qwisp_b200.tell import SpecStats, speculative_greedy
    prompt, n_new = [1, 2, 3, 1, 2], 120
    plain = ToyBackend()
    want = [plain.step_argmax(prompt)[-1]]
    while len(want) < n_new:
        want.append(plain.step_argmax([want[-1]])[0])
    stats = SpecStats()
    spec = ToyBackend()
    got = speculative_greedy(spec, prompt, n_new, chunk=2, stats=stats)
    assert got == want
    assert stats.accepted > 0 and stats.rollbacks > 0 and stats.verify_calls > stats.rollbacks
    assert stats.verify_calls + stats.single_steps < n_new           # fewer model calls than tokens
