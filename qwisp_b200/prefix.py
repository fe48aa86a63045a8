"""Cross-request prefix cache, RAM tier: whole decode states keyed by token content
(`PrefixRAMStore`, swift/Sources/QwispCore/PrefixPersist.swift:196-235).

An entry is (tokens, state blob) where the blob is a stream's persistent state
(`Stream.state_save`, the reference's persistentStateData) after exactly those tokens.  `save`
drops entries that are a prefix of the new key (earlier turns of the same conversation),
inserts most-recently-used first and evicts from the tail while the byte budget is exceeded;
`best_match` returns the entry whose key is the longest whole prefix of the content and marks
it most recently used.  A budget of 0 disables the store.

The disk tier below ("QWP1") keeps the same (tokens, blob) pairs in files, one per key, so that a
fresh process can restore them.
"""
import os
import struct


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

    def max_common_prefix(self, content):
        """Longest common token prefix between `content` and ANY stored key (a partial match, unlike best_match):
        evidence that a prefix recurs (PrefixPersist.swift:239-251).  Does not touch the MRU order."""
        best = 0
        for k, _ in self.entries:
            n = min(len(k), len(content))
            i = 0
            while i < n and k[i] == int(content[i]):
                i += 1
            best = max(best, i)
        return best

    def remove_all(self):
        self.entries = []


# ---------------------------------------------------------------------------------------------
# Disk tier ("QWP1", swift/Sources/QwispCore/PrefixPersist.swift:19-160)
# ---------------------------------------------------------------------------------------------
QWP1_MAGIC = 0x31505751          # "QWP1" little-endian
QWP1_FORMAT = 1


def fnv1a64(data):
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x00000100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def qwp1_encode(model, tokens, state):
    """magic | format | modelLen u32 | model utf8 | tokenCount u32 | tokens int32 LE | state blob (PrefixPersist.swift:61-74)."""
    m = model.encode("utf-8")
    toks = struct.pack(f"<{len(tokens)}i", *[int(t) for t in tokens])
    return struct.pack("<III", QWP1_MAGIC, QWP1_FORMAT, len(m)) + m + struct.pack("<I", len(tokens)) + toks + bytes(state)


def qwp1_decode(data, want_state=True):
    """-> (model, tokens, state) or None on any malformed header (PrefixPersist.swift:76-96)."""
    try:
        if len(data) < 12:
            return None
        magic, fmt, ml = struct.unpack_from("<III", data, 0)
        off = 12
        if magic != QWP1_MAGIC or fmt != QWP1_FORMAT or len(data) < off + ml + 4:
            return None
        model = bytes(data[off:off + ml]).decode("utf-8")
        off += ml
        (tc,) = struct.unpack_from("<I", data, off)
        off += 4
        if len(data) < off + tc * 4:
            return None
        tokens = list(struct.unpack_from(f"<{tc}i", data, off))
        off += tc * 4
        return model, tokens, (bytes(data[off:]) if want_state else b"")
    except (struct.error, UnicodeDecodeError):
        return None


class PrefixDiskStore:
    """One file per (model, exact token prefix); any key mismatch invalidates; least recently used files
    (by mtime) are evicted beyond `max_slots` files or `store_budget` bytes; states above `max_bytes` are
    not written (PrefixPersist.swift:98-160)."""

    def __init__(self, directory, model, max_slots=20, max_bytes=512 << 20, store_budget=2048 << 20):
        self.dir, self.model = directory, model
        self.max_slots, self.max_bytes, self.store_budget = max(1, max_slots), max_bytes, store_budget
        self.restore_hits = 0

    def path(self, tokens):
        ident = self.model.encode("utf-8") + struct.pack(f"<{len(tokens)}i", *[int(t) for t in tokens])
        return os.path.join(self.dir, "prefix-%016x.bin" % fnv1a64(ident))

    def has(self, tokens):
        return os.path.exists(self.path(tokens))

    def save(self, tokens, state):
        if len(state) > self.max_bytes or not len(tokens):
            return
        os.makedirs(self.dir, exist_ok=True)
        p = self.path(tokens)
        if os.path.exists(p):                       # same key = same content: refresh the LRU stamp only
            os.utime(p, None)
            return
        tmp = p + ".tmp"
        with open(tmp, "wb") as f:
            f.write(qwp1_encode(self.model, tokens, state))
        os.replace(tmp, p)                          # atomic
        self.evict()

    def _bins(self):
        try:
            return [os.path.join(self.dir, n) for n in os.listdir(self.dir) if n.endswith(".bin")]
        except OSError:
            return []

    def best_match(self, content):
        content = [int(t) for t in content]
        best = None
        for p in self._bins():
            try:
                with open(p, "rb") as f:
                    head = f.read(12)
                    if len(head) < 12:
                        continue
                    ml = struct.unpack_from("<I", head, 8)[0]
                    rest = f.read(ml + 4)
                    if len(rest) < ml + 4:
                        continue
                    tc = struct.unpack_from("<I", rest, ml)[0]
                    if tc > len(content):
                        continue
                    dec = qwp1_decode(head + rest + f.read(tc * 4), want_state=False)   # header and tokens only
            except OSError:
                continue
            if dec is None or dec[0] != self.model:
                continue
            toks = dec[1]
            if len(toks) > (len(best[1]) if best else 0) and content[:len(toks)] == toks:
                best = (p, toks)
        if best is None:
            return None
        try:
            with open(best[0], "rb") as f:
                dec = qwp1_decode(f.read(), want_state=True)
        except OSError:
            return None
        if dec is None:
            return None
        os.utime(best[0], None)                     # LRU touch
        self.restore_hits += 1
        return dec[1], dec[2]

    def evict(self, budget=None):
        dated = []
        for p in self._bins():
            try:
                st = os.stat(p)
                dated.append((st.st_mtime_ns, p, st.st_size))
            except OSError:
                pass
        dated.sort()                                 # oldest first
        total = sum(s for _, _, s in dated)
        cap = self.store_budget if budget is None else budget
        while dated and (len(dated) > self.max_slots or total > cap):
            _, p, size = dated.pop(0)
            try:
                os.remove(p)
            except OSError:
                pass
            total -= size
