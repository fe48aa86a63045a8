"""CPU test of the expert-parallel exchange with two gloo ranks: the rules in qwisp_b200/ep.py and
the property the device path relies on -- every (row, k) pair output is produced by exactly one
rank and is zero elsewhere, so summing the ranks' buffers returns each value bit for bit and the
owner can then combine in ascending k exactly as one GPU does."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from qwisp_b200 import ep
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, K, B, H = 16, 4, 3, 64                        # experts, top_k, rows per rank, width
    T = world * B
    rng = np.random.default_rng(100 + rank)
    my_inds = np.stack([rng.choice(E, size=K, replace=False) for _ in range(B)]).astype(np.int32)
    gathered = [torch.zeros((B, K), dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(my_inds))
    inds = torch.cat(gathered).numpy()               # rank r's rows at offset r*B, as on the device
    assert np.array_equal(inds[rank * B:(rank + 1) * B], my_inds)
    e0, e1 = ep.expert_range(rank, world, E)
    # what "expert e applied to row t" yields: any deterministic fp16 table stands in for the kernels
    table = np.random.default_rng(7).standard_normal((E, T, H)).astype(np.float16)
    buf = np.zeros((T * K, H), dtype=np.float16)
    for t in range(T):
        for k in range(K):
            e = int(inds[t, k])
            assert ep.owner_of_expert(e, world, E) == e // (E // world)
            if e0 <= e < e1:
                buf[t * K + k] = table[e, t]
    summed = torch.from_numpy(buf.astype(np.float32))   # gloo reduces fp32; the values are fp16-exact and each has one non-zero term
    dist.all_reduce(summed)
    full = summed.numpy().astype(np.float16)
    want = np.stack([table[int(inds[t, k]), t] for t in range(T) for k in range(K)])
    lo, hi = ep.pair_slices(rank, B, K)
    ok = np.array_equal(full.view(np.uint16)[lo:hi], want.view(np.uint16)[lo:hi]) and ep.streams_of_rank(rank, world, T) == list(range(rank * B, (rank + 1) * B))
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_two_rank_exchange_is_exact():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29610 + (os.getpid() % 200)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def test_partition_rules():
    from qwisp_b200 import ep
    assert ep.expert_range(3, 8, 256) == (96, 128)
    assert ep.streams_of_rank(1, 4, 64) == list(range(16, 32))
    assert ep.pair_slices(2, 8, 8) == (128, 192)
    with pytest.raises(ValueError):
        ep.expert_range(0, 3, 256)
