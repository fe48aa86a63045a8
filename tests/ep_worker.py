"""One rank of the expert-parallel check (launched by tests/test_gpu_ep.py through torch.distributed.run).
Every rank builds the same seeded model twice: one engine in expert-parallel mode, one plain.
Rank r owns streams r*B .. r*B+B-1 of a global set with seeded prompts; after a rank-local
prefill, S batched decode steps run on both engines.  The expert-parallel tokens must equal the
single-GPU tokens bit for bit."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import qwisp_b200 as Q

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")                   # host channel for the NCCL id only
    B, S, PROMPT = int(os.environ.get("EP_ROWS_PER_RANK", "4")), 6, 12
    geo = dict(hidden=2048, n_layers=4, attn_every=2, vocab=1024, n_experts=16, top_k=8, moe_inter=512,
               max_rows=max(32, world * B), max_streams=2 * B + 2, kv_page_size=32, kv_pages=4 * B + 16)
    cfg = Q.config(**geo)
    ep = Q.Engine.synthetic(cfg, seed=3, norm_jitter=0.1, conv_std=0.5)
    ref = Q.Engine.synthetic(cfg, seed=3, norm_jitter=0.1, conv_std=0.5)
    uid = torch.from_numpy(Q.Engine.ep_unique_id() if rank == 0 else np.zeros(128, dtype=np.uint8))
    dist.broadcast(uid, 0)
    ep.ep_init(rank, world, uid.numpy(), B)

    streams_ep, streams_ref, last_ep, last_ref = [], [], [], []
    for i in range(B):
        g = rank * B + i
        prompt = Q.ops.synth_tokens(3, f"ep.prompt.{g}", PROMPT + (g % 3), cfg.vocab)
        se, sr = ep.stream(64), ref.stream(64)
        last_ep.append(int(se.step_argmax(prompt)[-1]))
        last_ref.append(int(sr.step_argmax(prompt)[-1]))
        streams_ep.append(se); streams_ref.append(sr)
    assert last_ep == last_ref, "rank-local prefill differs between the two engines"
    ok = True
    for step in range(S):
        dist.barrier()
        te = ep.batch_step_argmax(streams_ep, last_ep)
        tr = ref.batch_step_argmax(streams_ref, last_ref)
        if not np.array_equal(te, tr):
            ok = False
            print(f"rank {rank} step {step}: expert-parallel {te.tolist()} != single-GPU {tr.tolist()}", flush=True)
        last_ep, last_ref = [int(v) for v in te], [int(v) for v in tr]
    fault = ep.gpu_fault()
    flag = torch.tensor([1 if (ok and fault is None) else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_CHECK_OK" if int(flag) == 1 else "EP_CHECK_FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
