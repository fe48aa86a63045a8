"""Cross-request prefix cache, RAM tier: whole decode states keyed by token content
(`PrefixRAMStore`, swift/Sources/QwispCore/PrefixPersist.swift:196-235).

An entry is (tokens, state blob) where the blob is a stream's persistent state
(`Stream.state_save`, the reference's persistentStateData) after exactly those tokens.  `save`
drops entries that are a prefix of the new key (earlier turns of the same conversation),
inserts most-recently-used first and evicts from the tail while the byte budget is exceeded;
`best_match` returns the entry whose key is the longest whole prefix of the content and marks
it most recently used.  A budget of 0 disables the store.
"""


class PrefixRAMStore:
    def __init__(self, budget=0):
        self.budget = int(budget)
        self.entries = []                      # MRU first: (tuple(tokens), bytes-like state)

    @property
    def nbytes(self):
        return sum(len(s) for _, s in self.entries)

    def save(self, tokens, state):
        key = tuple(int(t) for t in tokens)
        if self.budget <= 0 or not key or len(state) > self.budget:
            return
        self.entries = [(k, s) for (k, s) in self.entries if not (len(k) <= len(key) and key[:len(k)] == k)]
        self.entries.insert(0, (key, state))
        while self.nbytes > self.budget:
            self.entries.pop()

    def best_match(self, content):
        content = tuple(int(t) for t in content)
        best = -1
        for i, (k, _) in enumerate(self.entries):
            if len(k) <= len(content) and (best < 0 or len(k) > len(self.entries[best][0])) and content[:len(k)] == k:
                best = i
        if best < 0:
            return None
        e = self.entries.pop(best)
        self.entries.insert(0, e)
        return e

    def remove_all(self):
        self.entries = []
