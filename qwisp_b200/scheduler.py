"""Continuous-batching scheduler over a BatchSlots engine: the reference's token-budget round
(`ContinuousScheduler.budgetedStep`, swift/Sources/QwispCore/ContinuousBatch.swift:184-268), as a
synchronous driver.

One round: (1) free slots take requests from the queue head, first come first served, and only
while the engine's aggregate KV gate (`can_admit`) lets the head in — a head that does not fit
blocks everything behind it; (2) the running slots' share of the token budget is reserved
(`token_budget - running`), the remainder pays for prefill of the admitted requests in order,
each `admit_step` call doing at least one whole chunk and being charged only what it consumed;
(3) requests whose prefill finished emit their first token and become running; (4) every running
slot gets exactly one batched decode step.  A stop token ends a request without being emitted;
`max_tokens` caps what is emitted.

The engine side is any object with `slot_count`, `can_admit(prompt_len, seq_budget)`,
`admit_step(prompt, slot, token_budget, seq_budget)`, `step(last)` and `release(slot)`
(`LaneBatchSlots` in `engine.py`; a scripted fake in the tests).
"""
from dataclasses import dataclass, field


@dataclass
class Request:
    prompt: list
    max_tokens: int
    stop: frozenset = frozenset()
    out: list = field(default_factory=list)      # emitted tokens
    finished: bool = False

    def _yield(self, tok):
        self.out.append(int(tok))

    def _finish(self):
        self.finished = True


@dataclass
class _Pend:
    req: Request
    pos: int
    slot: int


@dataclass
class _Active:
    req: Request
    produced: int
    last: int


class ContinuousScheduler:
    def __init__(self, slots, token_budget):
        if token_budget <= 0:
            raise ValueError("token_budget must be positive")
        self.slots = slots
        self.token_budget = token_budget
        self.queue = []
        self.pending = []
        self.active = [None] * slots.slot_count
        self.rounds = 0
        self.max_running = 0

    def submit(self, req):
        self.queue.append(req)
        return req

    def idle(self):
        return not self.queue and not self.pending and all(a is None for a in self.active)

    def _retire(self, slot, req):
        req._finish()
        self.active[slot] = None
        self.slots.release(slot)

    def round(self):
        """One scheduling round (ContinuousBatch.swift:184-268)."""
        B = self.slots.slot_count
        owned = {p.slot for p in self.pending}
        for b in range(B):
            if self.active[b] is not None or b in owned or not self.queue:
                continue
            head = self.queue[0]
            if not self.slots.can_admit(len(head.prompt), len(head.prompt) + 1 + head.max_tokens):
                break                                             # head-of-line wait, never skip ahead
            req = self.queue.pop(0)
            if req.max_tokens <= 0:
                req._finish()
                continue
            self.pending.append(_Pend(req, 0, b))
            owned.add(b)
        running = sum(a is not None for a in self.active)
        pool = self.token_budget - running
        still, activate = [], []
        for p in self.pending:
            if pool <= 0:
                still.append(p)
                continue
            seq_budget = len(p.req.prompt) + 1 + p.req.max_tokens
            r = self.slots.admit_step(p.req.prompt, p.slot, pool, seq_budget)
            if r[0] == "failed":
                p.req._finish()
                self.slots.release(p.slot)
            elif r[0] == "prefilling":
                pool -= r[1]
                still.append(_Pend(p.req, p.pos + r[1], p.slot))
            else:                                                 # ("done", first, consumed): charge the work done, not the prompt length
                pool -= r[2]
                activate.append((p.slot, p.req, r[1]))
        self.pending = still
        for slot, req, first in activate:
            if first in req.stop:
                req._finish()
                self.slots.release(slot)
                continue
            req._yield(first)
            if req.max_tokens == 1:
                req._finish()
                self.slots.release(slot)
            else:
                self.active[slot] = _Active(req, 1, int(first))
        self.rounds += 1
        self.max_running = max(self.max_running, sum(a is not None for a in self.active))
        if all(a is None for a in self.active):
            return
        out = self.slots.step([a.last if a is not None else None for a in self.active])
        for b in range(B):
            a = self.active[b]
            if a is None or out[b] is None:
                continue
            tok = int(out[b])
            if tok in a.req.stop:                                 # stop token: not emitted
                self._retire(b, a.req)
                continue
            a.req._yield(tok)
            a.produced += 1
            a.last = tok
            if a.produced >= a.req.max_tokens:
                self._retire(b, a.req)

    def run_to_completion(self, max_rounds=1 << 20):
        while not self.idle():
            if self.rounds >= max_rounds:
                raise RuntimeError("scheduler did not drain")
            before = (len(self.queue), len(self.pending), sum(a is not None for a in self.active), self.rounds)
            self.round()
            if before[1] == 0 and before[2] == 0 and self.queue and len(self.queue) == before[0]:
                raise RuntimeError("queue head can never be admitted")   # the engine was empty and the gate still refused the head
        return self.rounds
