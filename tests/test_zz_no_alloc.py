"""GPU test of the allocation-free lm_head+argmax entry point (sl_op_lm_head_argmax_static),
through the C ABI.  Its tokens must equal the greedy argmax (lowest index on ties) of the logits
the existing device GEMV entry point (sl_op_qmm4_device) returns for the same buffers, on two
calls in a row that reuse the fixed scratch array, and a row count beyond the array's limit
must be refused without a launch.  The file name keeps it last in collection order, so it also
runs after every other test has used the library in the same process."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

K, N = 2048, 8192
MAX_ROWS = 8


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _make_weights(torch, L, seed, N=N):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randint(0, 2 ** 31 - 1, (N, K // 8), generator=g, device="cuda", dtype=torch.int64).to(torch.int32)
    s = (torch.rand((N, K // 64), generator=g, device="cuda") * 0.01 + 0.002).to(torch.float16)
    b = (-(torch.rand((N, K // 64), generator=g, device="cuda") * 0.08)).to(torch.float16)
    tiles = N // 16
    wr = torch.empty(tiles * (K // 128) * 1024, dtype=torch.uint8, device="cuda")
    sr = torch.empty(tiles * (K // 128) * 128, dtype=torch.uint8, device="cuda")
    assert L.sl_op_repack_q4_device(_ptr(w), _ptr(s), _ptr(b), K, N, _ptr(wr), _ptr(sr), None) == 0
    torch.cuda.synchronize()
    return wr, sr


def test_static_scratch_argmax_matches_gemv_twice():
    import torch
    import qwisp_b200 as Q
    L = Q.lib()
    wr, sr = _make_weights(torch, L, 7)
    g = torch.Generator(device="cuda").manual_seed(11)
    for call, M in enumerate((MAX_ROWS, 3)):            # two calls in a row on the same scratch array
        x = torch.randn((M, K), generator=g, device="cuda").to(torch.float16)
        y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        tok = torch.full((M,), -1, dtype=torch.int32, device="cuda")
        assert L.sl_op_qmm4_device(_ptr(x), _ptr(wr), _ptr(sr), M, K, N, _ptr(y), None) == 0
        assert L.sl_op_lm_head_argmax_static(_ptr(x), _ptr(wr), _ptr(sr), M, K, N, _ptr(tok), None) == 0
        torch.cuda.synchronize()
        logits = y.cpu().numpy().astype(np.float32)
        assert np.isfinite(logits).all()
        want = np.argmax(logits, axis=1).astype(np.int32)          # first maximum = lowest index on ties
        got = tok.cpu().numpy()
        assert np.array_equal(got, want), (call, got, want)


def test_static_scratch_argmax_full_vocabulary():
    """The real vocabulary (151,936 rows): the grid is capped at the scratch array's 444 partial slots, so
    every CTA strides over many tiles and the final reduction reads 444 partials per row.  Two calls in a
    row (8 rows, then 1) against the argmax of the GEMV entry point's logits."""
    import torch
    import qwisp_b200 as Q
    L = Q.lib()
    NV = 151936
    wr, sr = _make_weights(torch, L, 13, N=NV)
    g = torch.Generator(device="cuda").manual_seed(17)
    for call, M in enumerate((MAX_ROWS, 1)):
        x = torch.randn((M, K), generator=g, device="cuda").to(torch.float16)
        y = torch.empty((M, NV), dtype=torch.float16, device="cuda")
        tok = torch.full((M,), -1, dtype=torch.int32, device="cuda")
        assert L.sl_op_qmm4_device(_ptr(x), _ptr(wr), _ptr(sr), M, K, NV, _ptr(y), None) == 0
        assert L.sl_op_lm_head_argmax_static(_ptr(x), _ptr(wr), _ptr(sr), M, K, NV, _ptr(tok), None) == 0
        torch.cuda.synchronize()
        logits = y.cpu().numpy().astype(np.float32)
        assert np.isfinite(logits).all()
        want = np.argmax(logits, axis=1).astype(np.int32)
        got = tok.cpu().numpy()
        assert np.array_equal(got, want), (call, got, want)


def test_static_scratch_argmax_matches_cpu_oracle():
    """The same entry point against the CPU oracle's 4-bit product on seeded weights: identical tokens on
    every row whose top-1 / top-2 margin is clear of fp16 rounding."""
    import torch
    import qwisp_b200 as Q
    from oracle import oracle as O
    L = Q.lib()
    packed, scales, biases = O.synth_q4(21, "noalloc.w", N, K)
    x = O.synth_f16(21, "noalloc.x", MAX_ROWS * K).reshape(MAX_ROWS, K)
    ref = O.qmm4(x, packed, scales, biases).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).cuda()
    dw, ds, db, dx = dev(packed), dev(scales), dev(biases), dev(x)
    wr = torch.empty((N // 16) * (K // 128) * 1024, dtype=torch.uint8, device="cuda")
    sr = torch.empty((N // 16) * (K // 128) * 128, dtype=torch.uint8, device="cuda")
    assert L.sl_op_repack_q4_device(_ptr(dw), _ptr(ds), _ptr(db), K, N, _ptr(wr), _ptr(sr), None) == 0
    tok = torch.full((MAX_ROWS,), -1, dtype=torch.int32, device="cuda")
    assert L.sl_op_lm_head_argmax_static(_ptr(dx), _ptr(wr), _ptr(sr), MAX_ROWS, K, N, _ptr(tok), None) == 0
    torch.cuda.synchronize()
    got = tok.cpu().numpy()
    srt = np.sort(ref, axis=1)
    clear = (srt[:, -1] - srt[:, -2]) > 8e-3
    assert clear.any()
    assert np.array_equal(got[clear], np.argmax(ref, axis=1)[clear])
    assert ((got >= 0) & (got < N)).all()


def test_static_scratch_rejects_rows_beyond_limit():
    import torch
    import qwisp_b200 as Q
    L = Q.lib()
    wr, sr = _make_weights(torch, L, 9)
    M = MAX_ROWS + 1
    x = torch.zeros((M, K), dtype=torch.float16, device="cuda")
    tok = torch.full((M,), -7, dtype=torch.int32, device="cuda")
    rc = L.sl_op_lm_head_argmax_static(_ptr(x), _ptr(wr), _ptr(sr), M, K, N, _ptr(tok), None)
    torch.cuda.synchronize()
    from qwisp_b200._lib import SL_ERR_CAPACITY
    assert rc == SL_ERR_CAPACITY
    assert (tok.cpu().numpy() == -7).all()               # nothing was launched
