"""GPU tests of the one-kernel decode step (one cooperative launch per token: weight ring fed by bulk
copies, flag-in-data exchange between the phases) against the kernel-per-phase assembly it replaces for
single-stream decode.  Both assemblies run the same arithmetic, so tokens AND the caches they leave (KV
pages, GDN state, conv history: the QWS1 blob) must be identical bit for bit."""
import numpy as np
import pytest

from conftest import MINI, SEED, TINY, gpu_engine

pytestmark = pytest.mark.gpu


def _prompt(vocab, n, name):
    from oracle import oracle as O
    return O.synth_tokens(SEED, name, n, vocab)


@pytest.mark.parametrize("geom_name", ["tiny", "mini"])
def test_step_kernel_equals_kernel_per_phase(geom_name, tiny_engine, mini_engine):
    eng = tiny_engine if geom_name == "tiny" else mini_engine
    geom = TINY if geom_name == "tiny" else MINI
    assert eng.use_persistent(True), "the one-kernel step should be available for this geometry on a B200"
    try:
        p = _prompt(geom["vocab"], 7, "stepk")
        a, b = eng.stream(64), eng.stream(64)
        fa = int(a.step_argmax(p)[-1])
        fb = int(b.step_argmax(p)[-1])
        assert fa == fb
        K = 12
        eng.use_persistent(True)
        ta = a.chained_step_argmax(fa, K)
        eng.use_persistent(False)
        tb = b.chained_step_argmax(fb, K)
        assert eng.gpu_fault() is None
        assert list(ta) == list(tb), (list(ta), list(tb))
        assert np.array_equal(a.state_save(), b.state_save())
        # single steps through the host call, assemblies swapped: still identical
        eng.use_persistent(False)
        sa = [int(a.step_argmax([int(ta[-1])])[0])]
        eng.use_persistent(True)
        sb = [int(b.step_argmax([int(tb[-1])])[0])]
        for _ in range(3):
            eng.use_persistent(True)
            sa.append(int(a.step_argmax([sa[-1]])[0]))
            eng.use_persistent(False)
            sb.append(int(b.step_argmax([sb[-1]])[0]))
        assert sa == sb
        assert np.array_equal(a.state_save(), b.state_save())
        # a verify batch (several rows, kernel-per-phase) on top of step-kernel history == sequential single steps
        eng.use_persistent(True)
        rows = _prompt(geom["vocab"], 5, "stepk.rows")
        va = a.step_argmax(rows)
        vb = np.array([int(b.step_argmax([int(t)])[0]) for t in rows])
        assert np.array_equal(va, vb)
        assert np.array_equal(a.state_save(), b.state_save())
        a.close(); b.close()
    finally:
        eng.use_persistent(False)


def test_step_kernel_two_streams_interleaved(tiny_engine):
    """Two streams taking turns: the step kernel keeps nothing between launches except what is in the caches."""
    eng = tiny_engine
    V = TINY["vocab"]
    try:
        s1, s2, r1, r2 = (eng.stream(64) for _ in range(4))
        p1, p2 = _prompt(V, 4, "il1"), _prompt(V, 9, "il2")
        c1, c2 = int(s1.step_argmax(p1)[-1]), int(s2.step_argmax(p2)[-1])
        d1, d2 = int(r1.step_argmax(p1)[-1]), int(r2.step_argmax(p2)[-1])
        for _ in range(6):
            eng.use_persistent(True)
            c1 = int(s1.step_argmax([c1])[0]); c2 = int(s2.step_argmax([c2])[0])
            eng.use_persistent(False)
            d1 = int(r1.step_argmax([d1])[0]); d2 = int(r2.step_argmax([d2])[0])
            assert (c1, c2) == (d1, d2)
        assert np.array_equal(s1.state_save(), r1.state_save()) and np.array_equal(s2.state_save(), r2.state_save())
        for s in (s1, s2, r1, r2):
            s.close()
    finally:
        eng.use_persistent(False)


def test_step_kernel_full_model_tokens_identical():
    """The full synthetic 35B-A3B-shaped model: 16 chained tokens after a short prompt, both assemblies."""
    import qwisp_b200 as Q
    cfg = Q.config(max_rows=16, max_streams=2, kv_page_size=64, kv_pages=8)
    eng = Q.Engine.synthetic(cfg, seed=0, norm_jitter=0.0, conv_std=0.02)
    try:
        assert eng.use_persistent(True)
        p = Q.ops.synth_tokens(0, "bench.prompt", 12, cfg.vocab)
        a, b = eng.stream(64), eng.stream(64)
        fa, fb = int(a.step_argmax(p)[-1]), int(b.step_argmax(p)[-1])
        assert fa == fb
        eng.use_persistent(True)
        ta = a.chained_step_argmax(fa, 16)
        eng.use_persistent(False)
        tb = b.chained_step_argmax(fb, 16)
        assert eng.gpu_fault() is None
        assert list(ta) == list(tb), (list(ta), list(tb))
        assert np.array_equal(a.state_save(), b.state_save())
        a.close(); b.close()
    finally:
        eng.close()
