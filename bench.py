#!/usr/bin/env python
"""Benchmark of the Seedless decode core on B200.

Metric (BASELINE.json): decode tok/s at batch 1 -- the synthetic 35B-A3B-shaped model
(40 layers, 3 GDN : 1 full attention, 256-expert top-8 MoE + shared expert, 4-bit group-64
weights, vocab 151936), a 512-token random prompt, then greedy decode.  One "step" is one
decode step (one token per stream).  Timing follows the reference: decode only, prefill
excluded (swift/Sources/QwispCore/TellRuntime.swift:1267, 1449-1450).

  value  -- K chained decode steps enqueued back to back with the token fed back on the device,
            timed with CUDA events on the launching stream (inputs already resident in HBM)
  e2e    -- the same K steps through the step call a host runtime makes (host token in,
            host token out, a synchronisation every step), wall clock
  roofline     -- the kernel with the largest share of the step, timed live with CUDA events
  cpu_baseline -- the CPU oracle on the host cores, on a bounded sample of the same workload

`--impl reference` times the reference's path on the host cores instead (the CPU restatement of
its kernels: the reference itself is Swift + Metal and cannot run on Linux).
With N > 1 the workload is the batched one BASELINE.json pairs with multi-GPU: 64 concurrent streams
decoded with the MoE expert-parallel across the N GPUs (NCCL all-gather dispatch + reduce-scatter
combine per layer, attention/GDN data-parallel), aggregate tok/s, total work fixed ("strong").
The N=1 line carries the same 64-stream workload on one GPU as `batch64_1gpu`, so both series
(batch 1, batch 64) have their one-GPU point.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 512
METRIC = "decode_tok_per_s_batch1"
WORKLOAD = ("cfg4: synthetic 35B-A3B-shaped model (40 layers 3:1 GDN:attention, 256 experts top-8 + shared, "
            "4-bit g64, vocab 151936), 512-token prompt then greedy decode, batch 1")


def algorithmic_bytes_per_token(ctx_len):
    """Bytes one decoded token must read/write: 4-bit weights incl. scales/biases, fp16 router,
    fp32 GDN state (read + write), KV cache at the given context."""
    H, I, V, E = 2048, 512, 151936, 256
    q = 0.5625
    gdn = (8192 + 4096 + 64) * H * q + H * 4096 * q
    att = (8192 + 512 + 512) * H * q + H * 4096 * q
    moe = 9 * 3 * I * H * q + E * H * 2 + H * 2
    weights = 30 * gdn + 10 * att + 40 * moe + V * H * q
    state = 30 * 32 * 128 * 128 * 4 * 2
    kv = 10 * 2 * 2 * 256 * 2 * ctx_len
    return weights + state + kv


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = set()
        for r in self.rows:
            for i, n in enumerate(names):
                if len(r) > 4 + i and r[4 + i].lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_oracle_sample(max_seconds, prompt_tokens=2):
    """Time the CPU oracle on a bounded sample: the full-size model with experts generated on
    first use; a short prompt, then as many greedy decode steps as fit the budget.  The sample
    runs twice on the same tokens: the first pass generates the routed experts it touches, the
    second pass is the timed one."""
    from oracle import oracle as O
    cfg = O.config()
    t0 = time.time()
    model = O.Model(cfg, 0, lazy_experts=True)
    build_s = time.time() - t0
    prompt = O.synth_tokens(0, "bench.prompt", prompt_tokens, cfg.vocab)
    warm = model.stream(64)
    t0 = time.time()
    first = int(warm.step(prompt)[-1])
    per_tok = max((time.time() - t0) / prompt_tokens, 1e-3)
    steps = int(max(2, min(16, (max_seconds / 2.2) / per_tok - prompt_tokens)))
    toks, cur = [], first
    for _ in range(steps):
        cur = int(warm.step([cur])[0]); toks.append(cur)
    timed = model.stream(64)
    timed.step(prompt)
    t0 = time.time()
    cur = first
    for k in range(steps):
        cur = int(timed.step([cur])[0])
        assert cur == toks[k]
    dt = time.time() - t0
    return {"value": steps / dt, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"full 40-layer model, {prompt_tokens}-token prompt then {steps} greedy decode steps (context {prompt_tokens}..{prompt_tokens + steps}), "
                      f"OpenMP on all host cores; model build {build_s:.1f}s excluded",
            "steps": steps, "seconds": dt}


def run_reference(args, rank, world):
    if rank != 0:
        return
    cb = cpu_oracle_sample(max_seconds=float(os.environ.get("SEEDLESS_REF_SECONDS", "90")))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": cb["steps"], "warmup": args.warmup, "ms_per_step": 1000.0 / cb["value"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference's kernels on the host cores (the reference is Swift + Metal)"},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


BATCH_STREAMS = 64
WORKLOAD64 = ("cfg5 (decode part): the same model, 64 concurrent streams, seeded random prompts of 128-256 tokens "
              "(BASELINE.json: 128-2048; shortened to bound prefill time, stated here), batched greedy decode; "
              "prefill, the shared-prefix cache and the scheduler are outside the timed region")


def measure_batch64(Q, torch, dist, rank, world, layers, K, W):
    """64 streams dealt to the ranks in blocks; every decode step is one sl_batch_step_argmax per rank
    (expert-parallel when world > 1).  Returns (aggregate tok/s by device events, by wall clock,
    ms per step, launches per step, tokens of this rank)."""
    import numpy as np
    from qwisp_b200 import ep as EP
    mine = EP.streams_of_rank(rank, world, BATCH_STREAMS)
    B = len(mine)
    max_prompt = 256
    seq = max_prompt + K + W + 8
    cfg = Q.config(n_layers=layers, max_rows=max(max_prompt, BATCH_STREAMS), max_streams=B + 1, kv_page_size=64,
                   kv_pages=(B + 1) * (seq // 64 + 2))
    eng = Q.Engine.synthetic(cfg, seed=0, norm_jitter=0.0, conv_std=0.02)
    tstream = torch.cuda.Stream()
    eng.set_cuda_stream(tstream.cuda_stream)
    if world > 1:
        uid = torch.from_numpy(Q.Engine.ep_unique_id() if rank == 0 else np.zeros(128, dtype=np.uint8)).cuda()
        dist.broadcast(uid, 0)
        eng.ep_init(rank, world, uid.cpu().numpy(), B)
    streams, last = [], []
    for g in mine:
        n = 128 + (g * 37) % 129
        prompt = Q.ops.synth_tokens(0, f"bench.batch.prompt.{g}", n, cfg.vocab)
        st = eng.stream(seq)
        last.append(int(st.step_argmax(prompt)[-1]))
        streams.append(st)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        last = [int(v) for v in eng.batch_step_argmax(streams, last)]
    n0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record(tstream)
    toks = []
    for _ in range(K):
        out = eng.batch_step_argmax(streams, last)       # host tokens in, host tokens out, one synchronisation per step
        last = [int(v) for v in out]
        toks.append(out.copy())
    ev1.record(tstream)
    barrier()
    wall = time.time() - t0
    ms = ev0.elapsed_time(ev1)
    launches = (eng.launch_count() - n0) / K
    if dist is not None:
        t = torch.tensor([ms, wall * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1]) / 1e3
    fault = eng.gpu_fault()
    for st in streams:
        st.close()
    eng.close()
    if fault:
        raise SystemExit(f"engine fault during the batched run: {fault}")
    return {"tok_s": BATCH_STREAMS * K / (ms * 1e-3), "tok_s_wall": BATCH_STREAMS * K / wall, "ms_per_step": ms / K,
            "launches_per_step": launches, "rows_per_rank": B, "tokens": np.stack(toks)}


def run_batch64_line(args, rank, local_rank, world):
    # libraries (NCCL's version banner, for one) write to stdout: keep the descriptor for the one JSON line
    # and send everything else printed meanwhile to stderr
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    import torch
    import qwisp_b200 as Q
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    sampler.start()
    r = measure_batch64(Q, torch, dist, rank, world, args.layers, K, W)
    clocks = sampler.stop()
    if rank == 0:
        line = {"metric": "decode_tok_per_s_batch64_ep", "value": r["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD64 if args.layers == 40 else f"DEBUG {args.layers}-layer variant of " + WORKLOAD64,
                           "parallelism": f"ep{world}: experts split {256 // world} per GPU, {r['rows_per_rank']} streams per GPU; "
                                          "per MoE layer one NCCL all-gather (rows + routing) and one reduce-scatter (pair outputs)",
                           "l2": "inputs larger than L2: a step streams the touched experts (GBs) plus 1.6 GB of dense weights",
                           "timing": "K host-driven batched steps between CUDA events on the launching stream, max over ranks"},
                "clocks": clocks,
                "e2e": {"value": r["tok_s_wall"], "unit": "tok/s", "h2d_bytes_per_step": 4 * r["rows_per_rank"], "d2h_bytes_per_step": 4 * r["rows_per_rank"]},
                "gpu_launches": int(r["launches_per_step"] * K), "roofline": None, "cpu_baseline": None}
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    dist.destroy_process_group()
    os.close(json_fd)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batch64", action="store_true", help="skip the 64-stream measurement on the one-GPU line")
    ap.add_argument("--layers", type=int, default=40, help="debug only: fewer layers (the reported line then says so)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    if world > 1:
        return run_batch64_line(args, rank, local_rank, world)

    import numpy as np
    import torch
    import qwisp_b200 as Q

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    K, W = args.steps, max(args.warmup, 3)
    max_seq = PROMPT_LEN + 2 * (K + W) + 64
    cfg = Q.config(n_layers=args.layers, max_rows=PROMPT_LEN, max_streams=2, kv_page_size=64, kv_pages=2 * (max_seq // 64 + 2))
    eng = Q.Engine.synthetic(cfg, seed=0, norm_jitter=0.0, conv_std=0.02)
    tstream = torch.cuda.Stream()
    eng.set_cuda_stream(tstream.cuda_stream)
    prompt = Q.ops.synth_tokens(0, "bench.prompt", PROMPT_LEN, cfg.vocab)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident arm: chained decode ----
    st = eng.stream(max_seq)
    first = int(st.step_argmax(prompt)[-1])
    warm = st.chained_step_argmax(first, W)
    launches0 = eng.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(tstream):
        ev0.record(tstream)
        st.chained_enqueue(int(warm[-1]), K)
        ev1.record(tstream)
    barrier()
    clocks = sampler.stop()
    dev_ms = ev0.elapsed_time(ev1)
    toks_dev = st.chained_collect(K)
    launches_per_step = None

    # ---- end-to-end arm: one host call per token ----
    st2 = eng.stream(max_seq)
    cur = int(st2.step_argmax(prompt)[-1])
    for _ in range(W):
        cur = int(st2.step_argmax([cur])[0])
    barrier()
    t0 = time.perf_counter()
    toks_e2e = []
    for _ in range(K):
        cur = int(st2.step_argmax([cur])[0]); toks_e2e.append(cur)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    identical = bool(np.array_equal(np.asarray(toks_e2e), toks_dev))

    if dist is not None:
        t = torch.tensor([dev_ms, e2e_s * 1e3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    else:
        e2e_ms = e2e_s * 1e3

    # ---- per-kernel shares and the roofline of the dominant kernel (eager launches, CUDA events) ----
    roofline, shares = None, {}
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    if rank == 0:
        eng.use_graphs(False)
        cur2 = int(st.step_argmax([int(toks_dev[-1])])[0])
        n_before = eng.launch_count()
        eng.profile_start()
        nprof = 8
        for _ in range(nprof):
            cur2 = int(st.step_argmax([cur2])[0])
        rep = eng.profile_report()
        launches_per_step = (eng.launch_count() - n_before) // nprof
        eng.use_graphs(True)
        tot = sum(v[1] for v in rep.values())
        shares = {k: {"launches_per_step": v[0] // nprof, "ms_per_step": v[1] / nprof, "share": v[1] / tot} for k, v in rep.items()}
        dom = max((k for k in rep if rep[k][2] > 0), key=lambda k: rep[k][1])
        n, ms, by = rep[dom]
        # Average duration of one launch of the dominant kernel INSIDE the timed region: its share of
        # the step (per-launch CUDA events of the eager pass; ncu's launch list gives the same shares)
        # times the step time measured by the events around the timed region.  The eager per-launch
        # figure itself (event pair around every launch, no graph) is kept beside it.
        per_step = shares[dom]["launches_per_step"]
        us_in_step = shares[dom]["share"] * (dev_ms / K) / per_step * 1e3
        ach = (by / n) / (us_in_step * 1e-6) / 1e9
        # dram__bytes_read+write per launch from the ncu capture summarised in
        # profiles/decode_step_kernels_4layer_ncu_full.md (same weight shapes; k_gemv = mix of the
        # step's 30 GDN in/out projections and 10 attention q-k-v / o projections, the attention
        # in-projection scaled from the GDN one by its rows)
        ncu_traffic = {"k_gemv": (30 * 14.27e6 + 10 * 14.27e6 * 9216 / 12288 + 30 * 4.78e6 + 10 * 4.76e6) / 80,
                       "k_expert_gateup": 10.64e6, "k_expert_down": 5.36e6, "k_expert_fused": 10.64e6 + 5.36e6, "k_moe_router": 1.12e6, "k_gdn_core": 2.32e6 + 2.1e6}
        roofline = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs,
                    "traffic": ncu_traffic.get(dom) if args.layers == 40 else None, "peak_source": peak_src,
                    "algorithmic_bytes_per_launch": by / n, "us_per_launch": us_in_step, "us_per_launch_eager_events": ms / n * 1e3}

    tok_s = world * K / (dev_ms * 1e-3)
    e2e_tok_s = world * K / (e2e_ms * 1e-3)
    ctx = PROMPT_LEN + W + K // 2
    step_bytes = algorithmic_bytes_per_token(ctx) * (args.layers / 40.0 if args.layers != 40 else 1.0)
    step_gbs = step_bytes / (dev_ms / K * 1e-3) / 1e9

    cpu = None
    if rank == 0 and not args.no_cpu_baseline and args.layers == 40:
        cpu = cpu_oracle_sample(max_seconds=float(os.environ.get("SEEDLESS_CPU_SECONDS", "40")))
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    st.close(); st2.close(); eng.close()
    batch64 = None
    if not args.no_batch64:
        import torch as _t
        _t.cuda.empty_cache()
        b = measure_batch64(Q, torch, None, 0, 1, args.layers, min(K, 32), 3)
        batch64 = {"metric": "decode_tok_per_s_batch64", "value": b["tok_s"], "e2e": b["tok_s_wall"], "ms_per_step": b["ms_per_step"],
                   "steps": min(K, 32), "workload": WORKLOAD64, "launches_per_step": b["launches_per_step"]}
    if rank == 0:
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD if args.layers == 40 else f"DEBUG {args.layers}-layer variant of " + WORKLOAD,
                       "l2": "inputs larger than L2: each step streams ~1.7 GB of distinct weights (L2 is 126 MB)",
                       "parallelism": "batch-1 decode stays on one GPU; N>1 = one independent stream per GPU",
                       "prompt_len": PROMPT_LEN, "context_during_timing": [PROMPT_LEN + W, PROMPT_LEN + W + K],
                       "step_algorithmic_bytes": step_bytes, "step_achieved_gbs": step_gbs,
                       "step_frac_of_measured_hbm": step_gbs / peak_gbs, "step_frac_of_nominal_8tbs": step_gbs / 8000.0,
                       "device_vs_e2e_tokens_identical": identical, "kernel_shares": shares},
            "clocks": clocks,
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int((launches_per_step or 0) * K),
            "roofline": roofline, "cpu_baseline": cpu, "batch64_1gpu": batch64,
        }
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
