"""Greedy speculative decode over the backend closures, the way the reference's Tell runtime
drives its Seedless engine: a suffix-lookup draft from the token history
(swift/Sources/QwispCore/Tell.swift:104-175), one multi-row verify call, acceptance of the
matching prefix, and on a rejection a rollback followed by a replay of the accepted rows
(swift/Sources/QwispCore/TellRuntime.swift:716-900).  Greedy speculation never changes the
output: the token stream equals plain one-token-at-a-time greedy decode, which is what the
tests assert.  The module needs only a backend with `step_argmax(tokens) -> list`,
`snapshot()` and `rollback(snap)`; `qwisp_b200.engine.SpecBackend` is one."""


def suffix_draft(seq, max_match=8, draft_k=7, min_match=2, alpha=2):
    """Longest suffix of `seq` (between min_match and max_match tokens) that occurred earlier;
    the draft continues it by a vote among the earlier occurrences, most recent first on ties,
    keeping only the occurrences that agree with each chosen token.  At most
    min(draft_k, alpha * match_length) tokens."""
    n = len(seq)
    if n < min_match + 1:
        return []
    m = min(max_match, n - 1)
    while m >= min_match:
        pat = seq[n - m:]
        occ = [i for i in range(n - m - 1, -1, -1) if seq[i:i + m] == pat]      # most recent first
        if occ:
            cap = min(draft_k, alpha * m)
            draft, alive = [], occ
            while len(draft) < cap and alive:
                nxt = [seq[p + m + len(draft)] if p + m + len(draft) < n else -1 for p in alive]
                counts = {}
                for t in nxt:
                    if t >= 0:
                        counts[t] = counts.get(t, 0) + 1
                best, best_w = -1, -1
                for t in nxt:                       # most recent occurrence first; strict > keeps the earliest winner
                    if t >= 0 and counts[t] > best_w:
                        best, best_w = t, counts[t]
                if best < 0:
                    break
                draft.append(best)
                alive = [p for p, t in zip(alive, nxt) if t == best]
            return draft
        m -= 1
    return []


class SpecStats:
    def __init__(self):
        self.verify_calls = 0
        self.single_steps = 0
        self.drafted = 0
        self.accepted = 0
        self.rollbacks = 0


def speculative_greedy(backend, prompt, n_new, chunk=64, max_match=8, draft_k=7, min_match=2, alpha=2, stats=None):
    """Prefill `prompt` in chunks, then produce n_new greedy tokens with suffix-lookup speculation.
    Returns the new tokens.  `stats`, when given, counts calls and accepted drafts."""
    stats = stats if stats is not None else SpecStats()
    prompt = [int(t) for t in prompt]
    last = None
    for i in range(0, len(prompt), chunk):
        out = backend.step_argmax(prompt[i:i + chunk])
        if out is None:
            raise RuntimeError("backend failed during prefill")
        last = int(out[-1])
    history = list(prompt)
    new = [last]
    history.append(last)
    while len(new) < n_new:
        draft = suffix_draft(history, max_match, draft_k, min_match, alpha)
        draft = draft[:max(0, n_new - len(new) - 1)]
        if not draft:
            out = backend.step_argmax([history[-1]])
            if out is None:
                raise RuntimeError("backend failed")
            stats.single_steps += 1
            new.append(int(out[0])); history.append(int(out[0]))
            continue
        snap = backend.snapshot()
        rows = [history[-1]] + draft
        out = backend.step_argmax(rows)             # out[i] = the model's token after rows[:i+1]
        if out is None:
            raise RuntimeError("backend failed during verify")
        stats.verify_calls += 1
        stats.drafted += len(draft)
        acc = 0
        while acc < len(draft) and draft[acc] == int(out[acc]):
            acc += 1
        stats.accepted += acc
        if acc < len(draft):
            # the call advanced the caches by all rows: go back and replay the rows that stand
            backend.rollback(snap)
            stats.rollbacks += 1
            redo = backend.step_argmax(rows[:acc + 1])
            if redo is None or int(redo[-1]) != int(out[acc]):
                raise RuntimeError("replay after rollback disagrees with the verify call")
        got = draft[:acc] + [int(out[acc])]
        new.extend(got); history.extend(got)
    return new[:n_new]
