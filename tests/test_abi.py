"""The C-ABI library loads and exports every symbol include/seedless_b200.h declares; without a
GPU every entry point that needs one fails loudly (no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT, has_gpu


def header_symbols():
    hdr = open(os.path.join(ROOT, "include", "seedless_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(sl_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    from qwisp_b200 import _lib
    lib = _lib.lib()
    names = header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.SYMBOLS), "python binding table and header disagree"


def test_struct_layout_matches_header():
    from qwisp_b200 import _lib
    assert C.sizeof(_lib.SlConfig) == 18 * 4
    assert C.sizeof(_lib.SlSynthSpec) == 16
    assert C.sizeof(_lib.SlWeightDesc) == 32
    assert C.sizeof(_lib.SlSnap) == 16


def test_no_oracle_in_product():
    """The product package must not import or link the oracle."""
    pkg = os.path.join(ROOT, "qwisp_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


@pytest.mark.skipif(has_gpu(), reason="checks the no-device error path")
def test_fails_loudly_without_gpu():
    import qwisp_b200 as Q
    with pytest.raises(Q.SeedlessError) as ei:
        Q.Engine.synthetic(Q.config(n_layers=2, attn_every=2, vocab=1024, n_experts=16))
    assert ei.value.code == -2
    with pytest.raises(Q.SeedlessError):
        Q.ops.qmm4(np.zeros((1, 256), np.float16), np.zeros((16, 32), np.uint32), np.zeros((16, 4), np.float16), np.zeros((16, 4), np.float16))


def test_invalid_config_rejected():
    import qwisp_b200 as Q
    with pytest.raises(Q.SeedlessError) as ei:
        Q.Engine.synthetic(Q.config(hidden=1000))
    assert ei.value.code == -1


def test_token_generator_matches_oracle():
    import qwisp_b200 as Q
    from oracle import oracle as O
    a = Q.ops.synth_tokens(5, "prompt", 64, 151936)
    b = O.synth_tokens(5, "prompt", 64, 151936)
    assert (a == b).all()
