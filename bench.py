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
  roofline     -- the dominant kernel, timed live with CUDA events inside the timed region.  With the
                  one-kernel decode step (--step-kernel) that kernel IS the step: one launch per token,
                  algorithmic bytes = the token's 1.7 GB, duration = the events around the K launches / K.
                  With the kernel-per-phase assembly (the default) it is the kernel with the
                  largest share of a separate eager pass.
  cpu_baseline -- the CPU oracle on the host cores, on a bounded sample of the same workload

`--impl reference` times the reference's path on the host cores instead (the CPU restatement of
its kernels: the reference itself is Swift + Metal and cannot run on Linux).
With N > 1 the workload is the batched one BASELINE.json pairs with multi-GPU: 64 concurrent streams
decoded with the MoE expert-parallel across the N GPUs (dispatch and combine per layer by the library's own
kernels over NVLink peer memory, attention/GDN data-parallel), aggregate tok/s, total work fixed ("strong").
The N=1 line carries the same 64-stream workload on one GPU as `batch64_1gpu`, so both series
(batch 1, batch 64) have their one-GPU point.  It also carries
  prefill   -- a 4096-token prompt through the prefill-mode forward in 1024-token calls (tok/s, per-kernel shares)
  cfg5_1gpu -- BASELINE.json's continuous-batching configuration as a whole job: 64 requests through the
               token-budget scheduler and the lane slots with the shared-prefix store, wall clock; end-to-end and
               decode-only tok/s
(`--no-batch64`, `--no-prefill`, `--no-cfg5` skip them).  SEEDLESS_BENCH_TRACE=1 prints the stages of the batched
measurement with their times to stderr.
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


def batch_step_bytes_per_rank(streams_per_rank, world, ctx_len):
    """Algorithmic bytes one rank moves in a 64-stream decode step: the replicated dense weights once, the
    experts touched on this rank (EXPECTED distinct experts per layer for uniform routing of 64 x 8 picks over
    256, divided among the ranks -- stated as an expectation, the routing of the run is not read back), the
    rank's streams' GDN state (read + write) and KV."""
    H, I, V, E = 2048, 512, 151936, 256
    q = 0.5625
    gdn = (8192 + 4096 + 64) * H * q + H * 4096 * q
    att = (8192 + 512 + 512) * H * q + H * 4096 * q
    dense = 30 * gdn + 10 * att + 40 * (3 * I * H * q + E * H * 2 + H * 2) + V * H * q
    distinct = E * (1.0 - (1.0 - 1.0 / E) ** (BATCH_STREAMS * 8))
    experts = 40 * (distinct / world) * 3 * I * H * q
    state = streams_per_rank * 30 * 32 * 128 * 128 * 4 * 2
    kv = streams_per_rank * 10 * 2 * 2 * 256 * 2 * ctx_len
    return dense + experts + state + kv


def measured_traffic(kernel):
    """dram bytes per launch of `kernel` from the ncu capture summarised under profiles/ (a small JSON the
    summary's author writes next to it); None when there is no capture of the current kernel."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
        return t.get(kernel, {}).get("dram_bytes_per_launch")
    except (OSError, ValueError):
        return None


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


def cpu_oracle_sample(max_seconds, prompt_tokens=2, min_steps=2, max_steps=16):
    """Time the CPU oracle on a bounded sample: the full-size model with experts generated on
    first use; a short prompt, then as many greedy decode steps as fit the budget.  The sample
    runs twice on the same tokens: the first pass generates the routed experts it touches, the
    second pass is the timed one."""
    from oracle import oracle as O
    O.set_num_threads(os.cpu_count())
    cfg = O.config()
    t0 = time.time()
    model = O.Model(cfg, 0, lazy_experts=True)
    build_s = time.time() - t0
    prompt = O.synth_tokens(0, "bench.prompt", prompt_tokens, cfg.vocab)
    warm = model.stream(prompt_tokens + 2 * max_steps + 8)
    t0 = time.time()
    first = int(warm.step(prompt)[-1])
    prefill_s = time.time() - t0
    blob = warm.state_save()                                  # the timed pass starts from the same context without a second prefill
    t0 = time.time()
    cur = int(warm.step([first])[0])
    per_tok = max(time.time() - t0, 1e-3)
    steps = int(max(min_steps, min(max_steps, (max_seconds / 2.0) / per_tok)))
    toks = [cur]
    for _ in range(steps - 1):
        cur = int(warm.step([cur])[0]); toks.append(cur)
    timed = model.stream(prompt_tokens + 2 * max_steps + 8)
    assert timed.state_restore(blob)
    t0 = time.time()
    cur = first
    for k in range(steps):
        cur = int(timed.step([cur])[0])
        assert cur == toks[k]
    dt = time.time() - t0
    return {"value": steps / dt, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"full 40-layer model, {prompt_tokens}-token prompt then {steps} greedy decode steps (context {prompt_tokens}..{prompt_tokens + steps}), "
                      f"OpenMP on all host cores; model build {build_s:.1f}s and prefill {prefill_s:.1f}s excluded; the steps run twice on the same tokens "
                      f"(the first pass generates the routed experts it touches), the second pass is timed",
            "steps": steps, "seconds": dt}


def cpu_oracle_batch_sample(n_streams, prompt_tokens, steps):
    """The 64-stream batched decode on the CPU oracle, bounded: every stream gets a short seeded prompt, then
    `steps` rounds in which each stream decodes one token (the oracle has no batched step; a round is the
    streams one after another, each step using all host cores).  Returns aggregate tok/s of the rounds."""
    from oracle import oracle as O
    O.set_num_threads(os.cpu_count())        # (a torchrun worker's OpenMP runtime starts with one thread)
    cfg = O.config()
    t0 = time.time()
    model = O.Model(cfg, 0, lazy_experts=True)
    build_s = time.time() - t0
    streams, last = [], []
    for g in range(n_streams):
        st = model.stream(prompt_tokens + steps + 8)
        prompt = O.synth_tokens(0, f"bench.batch.prompt.{g}", prompt_tokens, cfg.vocab)
        last.append(int(st.step(prompt)[-1]))
        streams.append(st)
    for i, st in enumerate(streams):                       # one untimed round: generates the experts the timed rounds touch first
        last[i] = int(st.step([last[i]])[0])
    t0 = time.time()
    for _ in range(steps):
        for i, st in enumerate(streams):
            last[i] = int(st.step([last[i]])[0])
    dt = time.time() - t0
    return {"value": n_streams * steps / dt, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"full 40-layer model, {n_streams} streams with {prompt_tokens}-token prompts, {steps} timed rounds of one token per stream "
                      f"(context {prompt_tokens + 1}..{prompt_tokens + 1 + steps}), OpenMP on all host cores; model build {build_s:.1f}s, prompts and one warm-up round excluded",
            "steps": steps, "seconds": dt}


def run_reference(args, rank, world):
    """The reference's path on the host cores (its CPU restatement: the reference itself is Swift + Metal).
    N = 1: the batch-1 metric at the GPU arm's context (the 512-token prompt is prefilled on the CPU first).
    N > 1: the 64-stream batched metric on a bounded sample.  Rank 0 alone runs; under torchrun the other ranks exit."""
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: this arm is the CPU baseline, it uses every core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    if world > 1 or args.gpus > 1:
        cb = cpu_oracle_batch_sample(BATCH_STREAMS, prompt_tokens=int(os.environ.get("SEEDLESS_REF_BATCH_PROMPT", "4")), steps=max(1, min(args.steps, 2)))
        metric, workload, scaling = "decode_tok_per_s_batch64_ep", WORKLOAD64, "strong"
    else:
        cb = cpu_oracle_sample(max_seconds=float(os.environ.get("SEEDLESS_REF_SECONDS", "60")), prompt_tokens=PROMPT_LEN,
                               min_steps=max(2, min(args.steps, 8)), max_steps=max(2, min(args.steps, 16)))
        metric, workload, scaling = METRIC, WORKLOAD, "weak"
    line = {"impl": "reference", "metric": metric, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": cb["steps"], "warmup": args.warmup, "ms_per_step": 1000.0 / cb["value"] * (BATCH_STREAMS if metric.endswith("ep") else 1),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload, "note": "CPU restatement of the reference's kernels on the host cores (the reference is Swift + Metal); " + cb["sample"]},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


BATCH_STREAMS = 64
WORKLOAD64 = ("cfg5 (decode part): the same model, 64 concurrent streams, seeded random prompts of 128-256 tokens "
              "(BASELINE.json: 128-2048; shortened to bound prefill time, stated here), batched greedy decode; "
              "prefill, the shared-prefix cache and the scheduler are outside the timed region")


PREFILL_TOKENS = 4096


def measure_prefill(Q, torch, layers, n_tokens=PREFILL_TOKENS, chunk=1024, reps=3):
    """Prefill-mode forward (tensor-core GEMM for the dense projections) of one n_tokens prompt given as HOST
    tokens, in calls of `chunk` tokens (the engine's largest call); CUDA events on the engine's stream around each
    of `reps` passes after one warm-up pass, the stream reset between passes.  Also the per-kernel CUDA-event
    shares of one more pass."""
    cfg = Q.config(n_layers=layers, max_rows=chunk, max_streams=1, kv_page_size=64, kv_pages=n_tokens // 64 + 4)
    eng = Q.Engine.synthetic(cfg, seed=0, norm_jitter=0.0, conv_std=0.02)
    tstream = torch.cuda.Stream()
    eng.set_cuda_stream(tstream.cuda_stream)
    prompt = Q.ops.synth_tokens(0, "bench.prefill.prompt", n_tokens, cfg.vocab)
    st = eng.stream(n_tokens + 64)

    def one_pass():
        for i in range(0, n_tokens, chunk):
            st.forward_hybrid(prompt[i:i + chunk], want_hidden=False)

    one_pass()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        st.reset()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record(tstream)
        one_pass()
        ev1.record(tstream)
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1))
    st.reset()
    eng.profile_start()
    one_pass()
    rep = eng.profile_report()
    tot = sum(v[1] for v in rep.values()) or 1.0
    shares = {k: {"launches": v[0], "ms": v[1], "share": v[1] / tot} for k, v in rep.items()}
    fault = eng.gpu_fault()
    st.close(); eng.close()
    ms = sorted(times)[len(times) // 2]
    return {"metric": "prefill_tok_per_s", "value": n_tokens / (ms * 1e-3), "unit": "tok/s", "ms": ms, "tokens": n_tokens, "calls": n_tokens // chunk,
            "mode": "prefill mode (sl_forward_hybrid): dense projections and experts on tcgen05 GEMMs, router logits and attention on mma.sync tiles, GDN recurrence on the scan kernel",
            "kernel_shares": shares, "gpu_fault": fault}


CFG5_STREAMS, CFG5_DECODE, CFG5_BUDGET, CFG5_PREFIX = 64, 256, 4096, 1024
WORKLOAD_CFG5 = ("cfg5 as BASELINE.json states it, one GPU: 64 requests submitted at once to the continuous-batching scheduler "
                 "(64 slots, 4096-token budget per round, head-of-line admission on the KV page gate), 256 greedy tokens each; "
                 "even-numbered requests = one common seeded 1024-token prefix + a seeded tail of 128..1024 tokens, odd-numbered "
                 "requests = seeded random prompts of 128..2048 tokens; prompt chunks of 1024 tokens in prefill mode; the "
                 "conversation store (RAM, 1 GiB) keeps prompt-end states, whose keys are the evidence that a prefix recurs; the "
                 "shared-prefix store (RAM, 2 GiB) then captures the state at the exact shared boundary and later requests "
                 "restore it (host blobs, as in the reference)")


def measure_cfg5(Q, torch, layers):
    """The whole cfg5 job through ContinuousScheduler + LaneBatchSlots on one GPU, wall clock around run_to_completion
    (host tokens in, host tokens out).  Decode throughput = tokens emitted by batched decode steps / the time spent in
    them (each step ends with a synchronisation); end-to-end = all emitted tokens / wall clock."""
    import numpy as np
    rng = np.random.RandomState(5)
    lens = [int(rng.randint(128, 2049)) for _ in range(CFG5_STREAMS)]
    seq_cap = 2048 + CFG5_DECODE + 2
    pages = CFG5_STREAMS * (-(-seq_cap // 64) + 1)
    cfg = Q.config(n_layers=layers, max_rows=1024, max_streams=CFG5_STREAMS + 1, kv_page_size=64, kv_pages=pages)
    eng = Q.Engine.synthetic(cfg, seed=0, norm_jitter=0.0, conv_std=0.02)
    common = [int(t) for t in Q.ops.synth_tokens(0, "bench.cfg5.common", CFG5_PREFIX, cfg.vocab)]
    prompts = []
    for i in range(CFG5_STREAMS):
        if i % 2 == 0:
            tail = 128 + (lens[i] - 128) * (1024 - 128) // (2048 - 128)
            prompts.append(common + [int(t) for t in Q.ops.synth_tokens(0, f"bench.cfg5.tail.{i}", tail, cfg.vocab)])
        else:
            prompts.append([int(t) for t in Q.ops.synth_tokens(0, f"bench.cfg5.prompt.{i}", lens[i], cfg.vocab)])
    shared, conv = Q.PrefixRAMStore(budget=2 << 30), Q.PrefixRAMStore(budget=1 << 30)
    slots = Q.LaneBatchSlots(eng, CFG5_STREAMS, chunk=1024, default_seq_budget=seq_cap, shared_store=shared, prefix_store=conv,
                             hybrid=True, min_shared=1024)
    step_time = [0.0, 0, 0]
    inner_step = slots.step

    def timed_step(last):
        t0 = time.perf_counter()
        out = inner_step(last)
        step_time[0] += time.perf_counter() - t0
        step_time[1] += sum(t is not None for t in out)
        step_time[2] += 1
        return out
    slots.step = timed_step
    sched = Q.ContinuousScheduler(slots, CFG5_BUDGET)
    reqs = [sched.submit(Q.Request(prompt=p, max_tokens=CFG5_DECODE)) for p in prompts]
    launches0 = eng.launch_count()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rounds = sched.run_to_completion()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    emitted = sum(len(r.out) for r in reqs)
    fault = eng.gpu_fault()
    out = {"metric": "cfg5_tok_per_s", "e2e_tok_s": emitted / wall, "decode_tok_s": step_time[1] / step_time[0] if step_time[0] > 0 else None,
           "wall_s": wall, "decode_s": step_time[0], "decode_steps": step_time[2], "emitted_tokens": emitted, "rounds": rounds,
           "prompt_tokens": sum(len(p) for p in prompts), "prefilled_tokens": slots.prefilled_tokens, "restored_tokens": slots.restored_tokens,
           "prefix_captures": slots.captures, "prefix_restores": slots.restore_hits, "max_running": sched.max_running,
           "gpu_launches": int(eng.launch_count() - launches0), "all_finished": all(r.finished and len(r.out) == CFG5_DECODE for r in reqs),
           "gpu_fault": fault, "workload": WORKLOAD_CFG5}
    eng.close()
    return out


def measure_batch64(Q, torch, dist, rank, world, layers, K, W):
    """64 streams dealt to the ranks in blocks; every decode step is one sl_batch_step_argmax per rank
    (expert-parallel when world > 1).  Returns (aggregate tok/s by device events, by wall clock,
    ms per step, launches per step, tokens of this rank)."""
    import numpy as np
    from qwisp_b200 import ep as EP
    t_begin = time.time()
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
    streams, last, plens = [], [], []
    for g in mine:
        n = 128 + (g * 37) % 129
        prompt = Q.ops.synth_tokens(0, f"bench.batch.prompt.{g}", n, cfg.vocab)
        st = eng.stream(seq)
        last.append(int(st.step_argmax(prompt)[-1]))
        streams.append(st); plens.append(n)
    first_tokens = list(last)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    trace = (lambda msg: print(f"[bench rank {rank}] {msg} t={time.time() - t_begin:.1f}s", file=sys.stderr, flush=True)) if os.environ.get("SEEDLESS_BENCH_TRACE") else (lambda msg: None)
    trace("prompts done")
    warm_toks = []
    for _ in range(W):
        last = [int(v) for v in eng.batch_step_argmax(streams, last)]
        warm_toks.append(list(last))
        trace("warm-up step done")
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
    trace("timed steps done")
    launches = (eng.launch_count() - n0) / K
    if dist is not None:
        t = torch.tensor([ms, wall * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1]) / 1e3
    # per-kernel CUDA-event shares of a step (a few eager steps after the timed region; every rank runs them in lockstep)
    eng.use_graphs(False)
    prof_last = [int(v) for v in eng.batch_step_argmax(streams, last)]
    eng.profile_start()
    nprof = 3
    for _ in range(nprof):
        prof_last = [int(v) for v in eng.batch_step_argmax(streams, prof_last)]
    prep = eng.profile_report()
    eng.use_graphs(True)
    ptot = sum(v[1] for v in prep.values()) or 1.0
    kernel_shares = {k: {"launches_per_step": v[0] / nprof, "ms_per_step": v[1] / nprof, "share": v[1] / ptot} for k, v in prep.items()}
    fault = eng.gpu_fault()
    trace("profile pass done")
    for st in streams:
        st.close()
    # The batched (expert-parallel when world > 1) token streams against plain single-stream decoding of the same
    # prompts on this rank's engine (every rank holds all weights, and a single-stream step never uses the exchange):
    # the first two streams of the rank, every warm-up and timed step.
    identical = True
    all_toks = np.asarray(warm_toks + [list(t) for t in toks])          # [W + K, B]
    for j in range(min(2, B)):
        g = mine[j]
        solo = eng.stream(seq)
        cur = int(solo.step_argmax(Q.ops.synth_tokens(0, f"bench.batch.prompt.{g}", plens[j], cfg.vocab))[-1])
        identical = identical and (cur == first_tokens[j])
        for k in range(all_toks.shape[0]):
            cur = int(solo.step_argmax([cur])[0])
            identical = identical and (cur == int(all_toks[k, j]))
        solo.close()
    if dist is not None:
        t = torch.tensor([1 if identical else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        identical = bool(int(t[0]))
    fault = fault or eng.gpu_fault()
    eng.close()
    if fault:
        raise SystemExit(f"engine fault during the batched run: {fault}")
    return {"tok_s": BATCH_STREAMS * K / (ms * 1e-3), "tok_s_wall": BATCH_STREAMS * K / wall, "ms_per_step": ms / K,
            "launches_per_step": launches, "rows_per_rank": B, "tokens": np.stack(toks), "tokens_identical_to_solo": identical,
            "kernel_shares": kernel_shares,
            "ctx": float(np.mean(plens)) + W + K / 2.0}


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
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    cpu = None
    if rank == 0 and not args.no_cpu_baseline and args.layers == 40:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())          # torchrun exports 1; this leg is the CPU baseline
        cb = cpu_oracle_batch_sample(BATCH_STREAMS, prompt_tokens=2, steps=1)
        cpu = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        rank_bytes = batch_step_bytes_per_rank(r["rows_per_rank"], world, r["ctx"]) * (args.layers / 40.0 if args.layers != 40 else 1.0)
        rank_gbs = rank_bytes / (r["ms_per_step"] * 1e-3) / 1e9
        line = {"metric": "decode_tok_per_s_batch64_ep", "value": r["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD64 if args.layers == 40 else f"DEBUG {args.layers}-layer variant of " + WORKLOAD64,
                           "parallelism": f"ep{world}: experts split {256 // world} per GPU, {r['rows_per_rank']} streams per GPU; per MoE layer the normed rows "
                                          "and routing indices go to every rank and each pair's expert output goes back to its owner by this library's own "
                                          "kernels over NVLink peer memory (no collective inside a step; steps replay as CUDA graphs)",
                           "kernel_shares_rank0": r["kernel_shares"],
                           "l2": "inputs larger than L2: a step streams the touched experts (GBs) plus 1.6 GB of dense weights",
                           "timing": "K host-driven batched steps between CUDA events on the launching stream, max over ranks"},
                "clocks": clocks,
                "e2e": {"value": r["tok_s_wall"], "unit": "tok/s", "h2d_bytes_per_step": 4 * r["rows_per_rank"], "d2h_bytes_per_step": 4 * r["rows_per_rank"]},
                "gpu_launches": int(r["launches_per_step"] * K),
                "ep_tokens_identical": r["tokens_identical_to_solo"],
                "roofline": {"bound": "hbm", "kernel": "whole expert-parallel step (per rank)", "achieved": rank_gbs, "peak": peak_gbs, "unit": "GB/s",
                             "frac": rank_gbs / peak_gbs, "traffic": None, "algorithmic_bytes_per_step_per_rank": rank_bytes,
                             "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s",
                             "note": "per-rank bytes: replicated dense weights + expected distinct experts / ranks + the rank's streams' state and KV"},
                "cpu_baseline": cpu}
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
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill-mode measurement on the one-GPU line")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the continuous-batching job (scheduler + prefix store) on the one-GPU line")
    ap.add_argument("--step-kernel", action="store_true", help="batch-1 arm: decode with the one-kernel step instead of the kernel-per-phase assembly")
    ap.add_argument("--timeline", action="store_true", help="with --step-kernel: add the per-phase timeline of one step (median over CTAs, microseconds) to the line")
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
    cfg = Q.config(n_layers=args.layers, max_rows=PROMPT_LEN, max_streams=2, kv_page_size=64, kv_pages=2 * (max_seq // 64 + 2),
                   flags=Q._lib.SL_FLAG_STEP_KERNEL if args.step_kernel else 0)
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
    ctx = PROMPT_LEN + W + K // 2
    step_bytes = algorithmic_bytes_per_token(ctx) * (args.layers / 40.0 if args.layers != 40 else 1.0)
    persistent = eng.persistent_active()
    if rank == 0 and persistent:
        # the step is ONE launch of the step kernel: its duration is the timed region / K, measured by the events above
        us = dev_ms / K * 1e3
        ach = step_bytes / (us * 1e-6) / 1e9
        launches_per_step = 1
        shares = {"k_step_persistent": {"launches_per_step": 1, "ms_per_step": dev_ms / K, "share": 1.0}}
        roofline = {"bound": "hbm", "kernel": "k_step_persistent", "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs,
                    "traffic": measured_traffic("k_step_persistent") if args.layers == 40 else None, "peak_source": peak_src,
                    "algorithmic_bytes_per_launch": step_bytes, "us_per_launch": us,
                    "note": "one cooperative launch per token; duration = CUDA events around the K launches of the timed region / K"}
    elif rank == 0:
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
        # kernel-per-phase assembly: the dominant kernel's average duration inside the timed region = its share of
        # a step (per-launch CUDA events of an eager pass) times the step time measured by the events around the
        # timed region; the eager per-launch figure is kept beside it
        per_step = shares[dom]["launches_per_step"]
        us_in_step = shares[dom]["share"] * (dev_ms / K) / per_step * 1e3
        ach = (by / n) / (us_in_step * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs,
                    "traffic": measured_traffic(dom) if args.layers == 40 else None, "peak_source": peak_src,
                    "algorithmic_bytes_per_launch": by / n, "us_per_launch": us_in_step, "us_per_launch_eager_events": ms / n * 1e3}

    timeline = None
    if rank == 0 and persistent and args.timeline:
        # phase boundaries of the one-kernel step, stamped by every CTA with the global nanosecond timer: per layer
        # kind, the median over CTAs of each boundary relative to the median layer start, averaged over the layers
        names = ["start", "staged", "inproj_units", "inproj_stored", "mixer_end", "out_staged", "out_stored", "router_staged", "router_jobs_issued",
                 "routed", "gu_units", "gu_stored", "down_staged", "down_units", "layer_end", "logits_polled", "router_job_done"]
        cur3 = [int(toks_dev[-1])]

        def run3():
            for _ in range(3):
                cur3[0] = int(st.step_argmax([cur3[0]])[0])
        tl = eng.step_timeline(run3).astype(np.int64)
        tl = np.where(tl > 0, tl, -1).astype(np.float64)
        tl[tl < 0] = np.nan
        timeline = {"unit": "us, median over CTAs relative to the median layer start, mean over layers of the kind", "names": names}
        for kind, layers_of in (("gdn_layer", [L for L in range(args.layers) if (L + 1) % 4]), ("attention_layer", [L for L in range(args.layers) if (L + 1) % 4 == 0])):
            rows = []
            for L in layers_of[1:]:
                med = np.nanmedian(tl[:, L, :17], axis=0)
                rows.append((med - med[0]) / 1000.0)
            if rows:
                timeline[kind] = [round(float(x), 2) for x in np.nanmean(np.stack(rows), axis=0)]
        starts = np.nanmedian(tl[:, :, 0], axis=0)
        timeline["layer_us"] = {"gdn": round(float(np.mean([starts[L + 1] - starts[L] for L in range(args.layers - 1) if (L + 1) % 4])) / 1000.0, 2),
                                "attention": round(float(np.mean([starts[L + 1] - starts[L] for L in range(args.layers - 1) if (L + 1) % 4 == 0])) / 1000.0, 2) if args.layers >= 5 else None}
        head = np.nanmedian(tl[:, args.layers, :3], axis=0)
        timeline["lm_head_us"] = round(float(head[2] - head[0]) / 1000.0, 2)

    tok_s = world * K / (dev_ms * 1e-3)
    e2e_tok_s = world * K / (e2e_ms * 1e-3)
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
        bb = batch_step_bytes_per_rank(BATCH_STREAMS, 1, b["ctx"])
        bg = bb / (b["ms_per_step"] * 1e-3) / 1e9
        batch64 = {"metric": "decode_tok_per_s_batch64", "value": b["tok_s"], "e2e": b["tok_s_wall"], "ms_per_step": b["ms_per_step"],
                   "steps": min(K, 32), "workload": WORKLOAD64, "launches_per_step": b["launches_per_step"], "kernel_shares": b["kernel_shares"],
                   "roofline": {"bound": "hbm", "achieved": bg, "peak": peak_gbs, "unit": "GB/s", "frac": bg / peak_gbs, "traffic": None,
                                "algorithmic_bytes_per_step": bb, "note": "whole step; expert bytes are the expectation for uniform routing"}}
    prefill = None
    if not args.no_prefill:
        torch.cuda.empty_cache()
        prefill = measure_prefill(Q, torch, args.layers)
    cfg5 = None
    if not args.no_cfg5 and args.layers == 40:
        torch.cuda.empty_cache()
        cfg5 = measure_cfg5(Q, torch, args.layers)
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
                       "assembly": "one-kernel decode step (cooperative launch, weight ring, flag-in-data exchange)" if persistent else "kernel-per-phase (CUDA graph + programmatic dependent launch)",
                       "device_vs_e2e_tokens_identical": identical, "kernel_shares": shares, "step_timeline": timeline},
            "clocks": clocks,
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int((launches_per_step or 0) * K),
            "roofline": roofline, "cpu_baseline": cpu, "batch64_1gpu": batch64, "prefill": prefill, "cfg5_1gpu": cfg5,
        }
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
