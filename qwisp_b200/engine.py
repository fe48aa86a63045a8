"""Host-side mirror of the reference's engine interface over the C ABI.

`SpecBackend` carries the same members as the closure struct Tell drives
(swift/Sources/QwispCore/TellRuntime.swift:83-111): forward, stepArgmax, chainedStepArgmax,
stepLogitsRows, snapshot / rollback, fullSnapshot / fullRestore, persistentState /
restorePersistentState, gpuFault.  Failures follow the reference's convention: the call
returns None and `gpu_fault()` turns non-None (SeedlessFusedVerify.swift:388-416).
`LaneBatchSlots` mirrors `protocol BatchSlots` (ContinuousBatch.swift:38-66) the way
`LaneBatchSlots` implements it (LaneServe.swift:296-494): resumable chunked prefill per
slot, one batched greedy step over the active slots, release.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import SeedlessError, SlSnap, SlWeightDesc, lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Engine:
    """Weights + scratch + KV arena on one GPU (SeedlessEngine.build + makeFused)."""

    def __init__(self, cfg, handle):
        self.cfg = cfg
        self._h = handle

    @classmethod
    def synthetic(cls, cfg, seed=0, norm_jitter=0.0, conv_std=0.02):
        h = C.c_void_p()
        spec = _lib.synth_spec(seed, norm_jitter, conv_std)
        rc = lib().sl_engine_create_synthetic(C.byref(cfg), C.byref(spec), C.byref(h))
        if rc != 0:
            raise SeedlessError(rc, "sl_engine_create_synthetic")
        return cls(cfg, h)

    @classmethod
    def from_tensors(cls, cfg, tensors):
        """tensors: dict name -> contiguous numpy array in the MLX layout named in the header."""
        keep = [np.ascontiguousarray(v) for v in tensors.values()]
        descs = (SlWeightDesc * len(keep))()
        for i, (name, arr) in enumerate(zip(tensors.keys(), keep)):
            descs[i] = SlWeightDesc(name.encode(), arr.ctypes.data, arr.nbytes, 0)
        h = C.c_void_p()
        rc = lib().sl_engine_create(C.byref(cfg), descs, len(keep), C.byref(h))
        if rc != 0:
            raise SeedlessError(rc, "sl_engine_create")
        return cls(cfg, h)

    @classmethod
    def from_checkpoint(cls, cfg, paths):
        """Engine over safetensors shards in the reference's tensor naming (SeedlessEngine.swift:33-143)."""
        from .checkpoint import load_checkpoint
        return cls.from_tensors(cfg, load_checkpoint(paths, cfg.n_layers, cfg.attn_every))

    def close(self):
        if self._h:
            lib().sl_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, where):
        if rc != 0:
            raise SeedlessError(rc, where, self.gpu_fault())

    def gpu_fault(self):
        f = lib().sl_last_fault(self._h)
        return f.decode() if f else None

    def inject_fault(self, on=True):
        lib().sl_inject_fault(self._h, 1 if on else 0)

    def use_persistent(self, on=True):
        """Select the one-kernel decode step (True) or the kernel-per-phase assembly (the default) for
        single-stream decode steps; returns whether the one-kernel step is available."""
        return lib().sl_engine_use_persistent(self._h, 1 if on else 0) == 1

    def step_timeline(self, run):
        """Profile one or more one-kernel steps: arms the timeline, calls run(), returns the last step's stamps as
        uint32 [CTAs, layers + 1, 24] (nanoseconds since each CTA's start; 0 = not reached)."""
        G = lib().sl_debug_step_timeline(self._h, 1, None, 0)
        if G <= 0:
            raise SeedlessError(G, "sl_debug_step_timeline")
        run()
        out = np.zeros((G, self.cfg.n_layers + 1, 24), dtype=np.uint32)
        self._check(lib().sl_debug_step_timeline(self._h, 0, _ptr(out), out.size), "sl_debug_step_timeline")
        return out

    def persistent_active(self):
        return lib().sl_engine_use_persistent(self._h, -1) == 1

    def debug_wait_timeout(self):
        """Test hook: enqueue a kernel whose bounded wait runs out (nothing faults); the next call fails."""
        self._check(lib().sl_debug_wait_timeout(self._h), "sl_debug_wait_timeout")

    def set_cuda_stream(self, cuda_stream_handle):
        self._check(lib().sl_engine_set_cuda_stream(self._h, C.c_void_p(cuda_stream_handle)), "sl_engine_set_cuda_stream")

    def launch_count(self):
        return lib().sl_engine_launch_count(self._h)

    def use_graphs(self, on):
        self._check(lib().sl_engine_use_graphs(self._h, 1 if on else 0), "sl_engine_use_graphs")

    def profile_start(self):
        self._check(lib().sl_profile_start(self._h), "sl_profile_start")

    def profile_report(self):
        """-> {kernel: (launches, total_ms, algorithmic_bytes)} for the eager launches since profile_start()."""
        buf = C.create_string_buffer(1 << 16)
        self._check(lib().sl_profile_report(self._h, buf, len(buf)), "sl_profile_report")
        out = {}
        for line in buf.value.decode().splitlines():
            name, n, ms, by = line.split()
            out[name] = (int(float(n)), float(ms), float(by))
        return out

    def tensor_bytes(self, name):
        n = C.c_uint64()
        self._check(lib().sl_engine_tensor_bytes(self._h, name.encode(), C.byref(n)), "sl_engine_tensor_bytes")
        return n.value

    def read_tensor(self, name):
        n = self.tensor_bytes(name)
        buf = np.empty(n, dtype=np.uint8)
        self._check(lib().sl_engine_read_tensor(self._h, name.encode(), _ptr(buf), n), "sl_engine_read_tensor")
        return buf

    def stream(self, max_seq_len):
        h = C.c_void_p()
        self._check(lib().sl_stream_create(self._h, max_seq_len, C.byref(h)), "sl_stream_create")
        return Stream(self, h, max_seq_len)

    # ---- expert-parallel batched decode (one engine per GPU / process) ----
    @staticmethod
    def ep_unique_id():
        """128-byte NCCL id made on one rank; hand it to every rank's ep_init over any host channel."""
        buf = np.zeros(128, dtype=np.uint8)
        rc = lib().sl_ep_unique_id(_ptr(buf))
        if rc != 0:
            raise SeedlessError(rc, "sl_ep_unique_id", None)
        return buf

    def ep_init(self, rank, world, unique_id, rows_per_rank):
        """After this, batch_step_argmax with exactly rows_per_rank streams runs expert-parallel:
        this rank computes experts [rank*E/world, (rank+1)*E/world) for every rank's rows."""
        uid = np.ascontiguousarray(unique_id, dtype=np.uint8)
        assert uid.size == 128
        self._check(lib().sl_ep_init(self._h, int(rank), int(world), _ptr(uid), int(rows_per_rank)), "sl_ep_init")

    def lm_head_argmax(self, normed_rows):
        """arg-max token of the lm_head on already normed rows [M, hidden] (the first token after a prefill-mode prompt)."""
        from . import ops
        return ops.lm_head(self, normed_rows, want_logits=False)[1]

    def batch_step_argmax(self, streams, tokens):
        B = len(streams)
        arr = (C.c_void_p * B)(*[s._h for s in streams])
        toks = _i32(tokens)
        out = np.empty(B, dtype=np.int32)
        self._check(lib().sl_batch_step_argmax(self._h, arr, _ptr(toks), B, _ptr(out)), "sl_batch_step_argmax")
        return out


class Stream:
    """One sequence's caches: KV page table + GDN state."""

    def __init__(self, engine, handle, max_seq_len):
        self.engine = engine
        self._h = handle
        self.max_seq_len = max_seq_len

    def close(self):
        if self._h and self.engine._h:
            lib().sl_stream_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def length(self):
        return lib().sl_stream_len(self._h)

    def reset(self):
        self.engine._check(lib().sl_stream_reset(self._h), "sl_stream_reset")

    def forward(self, tokens, want_hidden=True):
        toks = _i32(tokens)
        out = np.empty((len(toks), self.engine.cfg.hidden), dtype=np.float16) if want_hidden else None
        self.engine._check(lib().sl_forward(self._h, _ptr(toks), len(toks), _ptr(out)), "sl_forward")
        return out

    def forward_hybrid(self, tokens, want_hidden=True):
        """Prefill-only forward (dense projections on the tensor cores); same outputs as forward()."""
        toks = _i32(tokens)
        out = np.empty((len(toks), self.engine.cfg.hidden), dtype=np.float16) if want_hidden else None
        self.engine._check(lib().sl_forward_hybrid(self._h, _ptr(toks), len(toks), _ptr(out)), "sl_forward_hybrid")
        return out

    def step_argmax(self, tokens):
        toks = _i32(tokens)
        out = np.empty(len(toks), dtype=np.int32)
        self.engine._check(lib().sl_step_argmax(self._h, _ptr(toks), len(toks), _ptr(out)), "sl_step_argmax")
        return out

    def chained_step_argmax(self, first, K):
        out = np.empty(K, dtype=np.int32)
        self.engine._check(lib().sl_chained_step_argmax(self._h, int(first), K, _ptr(out)), "sl_chained_step_argmax")
        return out

    def chained_enqueue(self, first, K):
        self.engine._check(lib().sl_chained_enqueue(self._h, int(first), K), "sl_chained_enqueue")

    def chained_collect(self, K):
        out = np.empty(K, dtype=np.int32)
        self.engine._check(lib().sl_chained_collect(self._h, K, _ptr(out)), "sl_chained_collect")
        return out

    def step_sample_rows(self, tokens, draft, inv_t, top_p, seed_lo, seed_hi, base_pos, logit_adj=None):
        """Forward the rows, then sample on the device: -> (full, resid, accept) int32 [M].
        logit_adj: optional f32 [vocab] added to every row's logits first (penalties + bias)."""
        toks = _i32(tokens)
        M = len(toks)
        d = None if draft is None else _i32(draft)
        adj = None if logit_adj is None else np.ascontiguousarray(logit_adj, dtype=np.float32)
        if adj is not None and adj.shape != (self.engine.cfg.vocab,):
            raise ValueError("logit_adj must have one entry per vocabulary token")
        full, resid, acc = (np.empty(M, dtype=np.int32) for _ in range(3))
        self.engine._check(lib().sl_step_sample_rows(self._h, _ptr(toks), M, _ptr(d) if d is not None else None,
                                                     _ptr(adj) if adj is not None else None, float(inv_t), float(top_p),
                                                     int(seed_lo), int(seed_hi), int(base_pos), _ptr(full), _ptr(resid), _ptr(acc)), "sl_step_sample_rows")
        return full, resid, acc

    def step_logits(self, tokens):
        toks = _i32(tokens)
        out = np.empty((len(toks), self.engine.cfg.vocab), dtype=np.float16)
        self.engine._check(lib().sl_step_logits(self._h, _ptr(toks), len(toks), _ptr(out)), "sl_step_logits")
        return out

    def snapshot(self):
        s = SlSnap()
        self.engine._check(lib().sl_snapshot(self._h, C.byref(s)), "sl_snapshot")
        return s

    def rollback(self, snap):
        self.engine._check(lib().sl_rollback_one_step(self._h, C.byref(snap)), "sl_rollback_one_step")

    def full_snapshot(self):
        h = C.c_void_p()
        self.engine._check(lib().sl_full_snapshot(self._h, C.byref(h)), "sl_full_snapshot")
        return FullSnapshot(h)

    def full_restore(self, snap):
        self.engine._check(lib().sl_full_restore(self._h, snap._h), "sl_full_restore")

    def state_save(self):
        n = C.c_uint64()
        self.engine._check(lib().sl_state_size(self._h, C.byref(n)), "sl_state_size")
        buf = np.empty(n.value, dtype=np.uint8)
        self.engine._check(lib().sl_state_save(self._h, _ptr(buf), n.value), "sl_state_save")
        return buf

    def state_restore(self, blob):
        """False on a malformed / mismatching blob: the caller must reset and cold-prefill."""
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        rc = lib().sl_state_restore(self._h, _ptr(blob), len(blob))
        if rc == _lib.SL_ERR_FORMAT:
            return False
        self.engine._check(rc, "sl_state_restore")
        return True


class FullSnapshot:
    def __init__(self, handle):
        self._h = handle

    def __del__(self):
        try:
            if self._h:
                lib().sl_fullsnap_free(self._h)
                self._h = None
        except Exception:
            pass


class SpecBackend:
    """The closure set Tell's speculative loop drives, bound to one stream."""

    def __init__(self, stream, hybrid_chunk=None):
        self.stream = stream
        # rows per prefill call: the library's own figure, min(1024, max_rows) (TellRuntime.swift:234-238), unless given
        chunk = lib().sl_hybrid_chunk(stream.engine._h)
        self.hybrid_chunk = min(hybrid_chunk, chunk) if hybrid_chunk else chunk

    def _guard(self, fn, *a):
        try:
            return fn(*a)
        except SeedlessError:
            return None

    def forward(self, tokens):
        return self._guard(self.stream.forward, tokens)

    def forward_hybrid(self, tokens):
        return self._guard(self.stream.forward_hybrid, tokens)

    def step_argmax(self, tokens):
        r = self._guard(self.stream.step_argmax, tokens)
        return None if r is None else [int(t) for t in r]

    def chained_step_argmax(self, first, K):
        r = self._guard(self.stream.chained_step_argmax, first, K)
        return None if r is None else [int(t) for t in r]

    def step_logits_rows(self, tokens):
        return self._guard(self.stream.step_logits, tokens)

    def snapshot(self):
        return self.stream.snapshot()

    def rollback(self, snap):
        self._guard(self.stream.rollback, snap)

    def full_snapshot(self):
        return self._guard(self.stream.full_snapshot)

    def full_restore(self, snap):
        self._guard(self.stream.full_restore, snap)

    def persistent_state(self):
        return self._guard(self.stream.state_save)

    def restore_persistent_state(self, blob):
        r = self._guard(self.stream.state_restore, blob)
        return bool(r)

    def gpu_fault(self):
        return self.stream.engine.gpu_fault()


class LaneAdmitPlan:
    """Where a new request starts and what it leaves behind (LaneServe.swift:98-131)."""

    def __init__(self, restore_len=0, capture_at=None, save_at_end=False):
        self.restore_len, self.capture_at, self.save_at_end = restore_len, capture_at, save_at_end

    def __eq__(self, o):
        return (self.restore_len, self.capture_at, self.save_at_end) == (o.restore_len, o.capture_at, o.save_at_end)

    def __repr__(self):
        return f"LaneAdmitPlan(restore_len={self.restore_len}, capture_at={self.capture_at}, save_at_end={self.save_at_end})"


def admit_plan(prompt_len, hit_len, lcp, min_shared):
    """hit_len: longest whole-entry store hit over prompt[:-1]; lcp: longest PARTIAL key match (two prompts sharing
    >= min_shared tokens define a recurring prefix).  The state is captured at the exact recurrence boundary only when
    that beats the restore point by more than a blob copy is worth (256 tokens of prefill) and leaves >= 1 token; the
    prompt-end state is saved unless the restore already covers everything but the last token
    (LaneServe.swift:117-131)."""
    capture = min(lcp, prompt_len - 1)
    if capture < min_shared or capture < hit_len + 256:
        capture = None
    save_at_end = prompt_len >= min_shared and hit_len < prompt_len - 1
    return LaneAdmitPlan(hit_len, capture, save_at_end)


class LaneBatchSlots:
    """BatchSlots over engine streams: resumable chunked prefill + batched greedy step (LaneServe.swift:331-485).

    hybrid: prompt chunks run in prefill mode (sl_forward_hybrid) and the first token is the arg-max of the lm_head on
    the last normed row, as the reference's lane prefill does; otherwise the strict forward.
    shared_store / prefix_store: optional PrefixRAMStore pair.  A new request restores the longest stored state whose
    tokens are a whole prefix of its prompt minus the last token, prefills only the rest, captures the state at the
    exact boundary where its prompt stops agreeing with a stored key (shared_store) and saves the prompt-end state
    (prefix_store, the reference's conversation store)."""

    def __init__(self, engine, slot_count, chunk=None, default_seq_budget=4096, prefix_store=None, shared_store=None,
                 hybrid=False, min_shared=1024):
        self.engine = engine
        self.slot_count = slot_count
        self.chunk = chunk or engine.cfg.max_rows
        self.default_seq_budget = default_seq_budget
        self.prefix_store = prefix_store
        self.shared_store = shared_store
        self.hybrid = hybrid
        self.min_shared = min_shared
        self.restored_tokens = 0
        self.restore_hits = 0
        self.captures = 0
        self.prefilled_tokens = 0
        self._streams = [None] * slot_count
        self._resume = [0] * slot_count
        self._plan = [None] * slot_count

    def can_admit(self, prompt_len, seq_budget):
        need = -(-max(seq_budget, prompt_len + 1) // self.engine.cfg.kv_page_size)
        used = sum(-(-s.max_seq_len // self.engine.cfg.kv_page_size) for s in self._streams if s is not None)
        return used + need <= self.engine.cfg.kv_pages

    def _stores(self):
        return [s for s in (self.shared_store, self.prefix_store) if s is not None and s.budget > 0]

    def _open(self, prompt, slot, seq_budget):
        self._streams[slot] = self.engine.stream(seq_budget or self.default_seq_budget)
        self._resume[slot] = 0
        self._plan[slot] = None
        plan = LaneAdmitPlan()
        stores = self._stores()
        if stores:
            matchable = prompt[:-1]
            hits = [h for h in (s.best_match(matchable) for s in stores) if h is not None]
            hit = max(hits, key=lambda h: len(h[0])) if hits else None
            lcp = max(s.max_common_prefix(prompt) for s in stores)
            plan = admit_plan(len(prompt), len(hit[0]) if hit else 0, lcp, self.min_shared)
            if plan.restore_len > 0:
                if self._streams[slot].state_restore(hit[1]):
                    self._resume[slot] = plan.restore_len        # restored tokens are not charged to the budget
                    self.restored_tokens += plan.restore_len
                    self.restore_hits += 1
                else:                                            # unusable blob: start cold on a fresh stream
                    self._streams[slot].close()
                    self._streams[slot] = self.engine.stream(seq_budget or self.default_seq_budget)
                    plan.restore_len = 0
        self._plan[slot] = plan

    def admit_step(self, prompt, slot, token_budget, seq_budget=0):
        """-> ("prefilling", consumed) | ("done", first_token, consumed) | ("failed",)"""
        try:
            if self._streams[slot] is None:
                self._open(prompt, slot, seq_budget)
            st, plan = self._streams[slot], self._plan[slot]
            pos = self._resume[slot]
            consumed = 0
            first = True
            while pos < len(prompt):
                end = min(pos + self.chunk, len(prompt))
                if plan.capture_at is not None and pos < plan.capture_at:
                    end = min(end, plan.capture_at)              # one chunk is split at the exact boundary
                n = end - pos
                if not first and consumed + n > token_budget:
                    break                                        # forward progress: at least one whole chunk per call
                last = (end == len(prompt))
                tok = None
                if self.hybrid:
                    normed = st.forward_hybrid(prompt[pos:end], want_hidden=last)
                    if last:
                        tok = int(self.engine.lm_head_argmax(normed[-1:])[0])
                elif last:
                    tok = int(st.step_argmax(prompt[pos:end])[-1])
                else:
                    st.forward(prompt[pos:end], want_hidden=False)
                pos = end
                consumed += n
                self.prefilled_tokens += n
                first = False
                if plan.capture_at is not None and pos == plan.capture_at and self.shared_store is not None:
                    self.shared_store.save(prompt[:pos], st.state_save())
                    self.captures += 1
                if last:
                    self._resume[slot] = pos
                    if plan.save_at_end and self.prefix_store is not None and self.prefix_store.budget > 0:
                        self.prefix_store.save(prompt, st.state_save())
                    return ("done", tok, consumed)
            self._resume[slot] = pos
            return ("prefilling", consumed)
        except SeedlessError:
            return ("failed",)

    def admit(self, prompt, slot):
        r = self.admit_step(prompt, slot, token_budget=1 << 30)
        return r[1] if r[0] == "done" else None

    def step(self, last):
        active = [b for b, t in enumerate(last) if t is not None]
        out = [None] * len(last)
        if not active:
            return out
        toks = self.engine.batch_step_argmax([self._streams[b] for b in active], [last[b] for b in active])
        for b, t in zip(active, toks):
            out[b] = int(t)
        return out

    def release(self, slot):
        if self._streams[slot] is not None:
            self._streams[slot].close()
            self._streams[slot] = None
        self._resume[slot] = 0
        self._plan[slot] = None
