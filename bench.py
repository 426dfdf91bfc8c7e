#!/usr/bin/env python
"""Headline benchmark: Q8_0 greedy decode on the Qwen3-0.6B-shaped decoder.

One "step" is one request of the reference's standard workload shape
(benchmarks/standard-v1.json:10-12: 512-token prompt, 256 greedy tokens, batch
1) on seeded synthetic Q8_0 weights.  Rank r of an N-GPU run serves its own
request on its own GPU (replicas, weak scaling, no data-path collective).

  value       decode tok/s with everything resident in HBM: the recorded decode
              graph replayed 255 times per request, CUDA events on the
              engine's stream, summed over ranks
  e2e         the same metric through the engine's public generate() call with
              host buffers: prompt ids uploaded, every token read back by the
              host (reference definition: (generated-1) / first->last token span)
  roofline    the Q8_0 GEMV launches of one decode step timed one dispatch each
              with CUDA events: algorithmic bytes / time against the measured
              HBM copy bandwidth
  cpu_baseline  the CPU oracle (a port of the reference's scalar executor) on a
              bounded sample of the same workload

`--impl reference` times that CPU port alone on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from tuckmill_b200 import testing as T  # noqa: E402

WORKLOADS = {
    "qwen3-0.6b": (T.QWEN3_0_6B, 512, 256),
    "gemma3-1b": (T.GEMMA3_1B, 512, 256),
    "qwen3-8b": (T.QWEN3_8B, 2048, 256),  # one sequence of the 8-GPU configuration's model (8.7 GB of Q8_0)
    "tiny-qwen3": (T.TINY_QWEN3, 32, 16),
}
METRIC = "q8_0_decode_tok_s"


def artifact(name: str, seed: int = 0) -> Path:
    shape = WORKLOADS[name][0]
    d = Path(os.environ.get("TUCKMILL_BENCH_DIR", "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"))
    path = d / f"tuckmill_{name}_seed{seed}.gguf"
    marker = path.with_suffix(".done")
    if not marker.exists():
        tmp = path.with_suffix(f".tmp{os.getpid()}")
        T.write_gguf(tmp, shape, seed=seed)
        os.replace(tmp, path)
        marker.write_text("ok")
    return path


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi SM clock / throttle reasons sampled during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._p, self._t = index, [], None, None

    def _run(self):
        for line in self._p.stdout:  # one line every 100 ms until the process is ended
            self.samples.append([c.strip() for c in line.strip().split(",")])

    def __enter__(self):
        try:
            self._p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                        "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                                       stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
            time.sleep(0.3)  # the first sample is there before the timed region starts
        except OSError:
            self._p = None
        return self

    def __exit__(self, *a):
        if self._p is not None:
            self._p.terminate()  # this process only
            try:
                self._p.wait(timeout=3)
            except subprocess.TimeoutExpired:
                self._p.kill()
            self._t.join(timeout=3)

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                mhz.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def cpu_leg(name: str, seed: int, decode_sample: int = 16, one_core_sample: int = 0):
    """Bounded sample of the workload on the CPU oracle, at the workload's own context length: the
    whole prompt is prefilled in 128-token chunks on all host threads (untimed), then `decode_sample`
    one-token greedy steps are timed at the positions right after it (the metric is decode tok/s).
    With `one_core_sample` > 0 that many further steps are timed on ONE thread -- the reference
    executor's own design (crates/tuckcore/src/executor.rs:813 is single-threaded).
    Returns (tok/s on all threads, threads, tok/s on one thread or None, description)."""
    import oracle as O

    O.build()
    shape, prompt_n, _ = WORKLOADS[name]
    path = artifact(name, seed)
    m = O.Model(path, kv_f16=True, threads=None)
    threads = m.threads
    m.reset(prompt_n + decode_sample + one_core_sample + 2)
    prompt = T.token_ids(seed, prompt_n, shape.vocab)
    logits = None
    for i in range(0, prompt_n, 128):
        logits = m.forward(prompt[i:i + 128], want_logits=i + 128 >= prompt_n)
    tok = O.argmax(logits)
    t0 = time.perf_counter()
    for _ in range(decode_sample):
        tok = O.argmax(m.forward([tok]))
    all_cores = decode_sample / (time.perf_counter() - t0)
    one_core = None
    if one_core_sample:
        m.threads = 1
        t0 = time.perf_counter()
        for _ in range(one_core_sample):
            tok = O.argmax(m.forward([tok]))
        one_core = one_core_sample / (time.perf_counter() - t0)
    sample = (f"{decode_sample} greedy decode steps at positions {prompt_n}..{prompt_n + decode_sample - 1} of the {name} "
              f"workload (its {prompt_n}-token prompt prefilled first, untimed)")
    return all_cores, threads, one_core, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape, prompt_n, decode_n = WORKLOADS[args.workload]
    vals, one = [], None
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        v, threads, one_core, sample = cpu_leg(args.workload, args.seed, decode_sample=12,
                                               one_core_sample=3 if i == args.warmup + args.steps - 1 else 0)
        if i >= args.warmup:
            vals.append(v)
        if one_core:
            one = one_core
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * (time.perf_counter() - t_all) / max(1, args.steps + args.warmup),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.workload, args.seed),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "cpu_baseline_1core": {"value": one, "unit": "tok/s", "cores": 1, "kind": "port",
                               "sample": "3 further decode steps of the same session on one thread"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def bench_config(workload: str, seed: int) -> dict:
    """The workload both arms name: the same keys and values in the CUDA line and the reference line."""
    shape, prompt_n, decode_n = WORKLOADS[workload]
    return {"workload": workload, "prompt_tokens": prompt_n, "decode_tokens": decode_n, "batch": 1, "kv": "f16",
            "weights": "Q8_0 random-init, seed %d" % seed}


def gemv_roofline(eng, shape, hbm_gbs, us_per_token, prompt_n):
    """Roofline of the dominant kernel of the timed region, the Q8_0 GEMV (every
    projection and the lm_head of a decode step are launches of it).

    Inside the replayed graph single launches cannot be bracketed by events, so
    the kernel's time within a step is the step's device time (measured over the
    timed region) times the GEMV's share of the step, the share taken from a
    pass that dispatches each operator on its own with events around it."""
    eng.reset()
    eng.prefill(T.token_ids(1, prompt_n, shape.vocab), want_token=True)  # the share is taken at the timed positions
    eng.decode_ungrouped(3)
    eng.fence()
    eng.profile(True)
    steps = 8
    eng.decode_ungrouped(steps)
    eng.fence()
    rows = {n: (ns, c) for n, ns, c in eng.profile_rows()}
    eng.profile(False)
    gemv_ns = sum(ns for n, (ns, c) in rows.items() if n.startswith("q8_0_gemv"))
    gemv_launches = sum(c for n, (ns, c) in rows.items() if n.startswith("q8_0_gemv"))
    total_ns = sum(ns for ns, c in rows.values())
    share = gemv_ns / total_ns
    # algorithmic bytes of the GEMV launches of one step: weights once, f32 in, f32 out
    per_step = shape.decode_weight_bytes()
    act = 0
    for _, o, i in shape.matrices(0):
        act += 4 * i + 4 * o
    per_step += act * shape.layers + 4 * shape.hidden + 4 * shape.vocab
    launches = gemv_launches / steps
    us_in_step = us_per_token * share
    achieved = per_step / (us_in_step * 1e3)  # bytes / ns == GB/s
    return {
        "bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
        "traffic": None, "kernel": "q8_gemv_kernel", "launches_per_step": launches,
        "bytes_per_launch": per_step / launches, "us_per_launch": us_in_step / launches,
        "gemv_share_of_step": share,
        "note": "0.6B-scale projections are 2-6 MB each: a launch is latency-bound, not bandwidth-bound; "
                "lm_head below is the one launch of the step that streams long enough to be",
        "by_operator_us_per_step_ungrouped": {n: round(ns / steps / 1e3, 2) for n, (ns, c) in sorted(rows.items())},
    }


def copy_bandwidth(torch, device):
    """Device-to-device copy of 1 GiB on THIS GPU (read + write bytes / time), the same kind of
    measurement the peak in MEASURED_PEAKS.json comes from: GPUs of this pool differ by 10-20 %."""
    n = 1 << 30
    a = torch.empty(n, dtype=torch.uint8, device=f"cuda:{device}")
    b = torch.empty_like(a)
    for _ in range(2):
        b.copy_(a)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        b.copy_(a)
    e1.record()
    torch.cuda.synchronize()
    gbs = 2.0 * n * 5 / (e0.elapsed_time(e1) * 1e-3) / 1e9
    del a, b
    return gbs


def lm_head_roofline(device, shape, hbm_gbs, torch):
    """The step's largest launch alone: the vocab x hidden GEMV, 20 launches in one
    replayed graph with events on its stream either side (the weights, 1.0625
    bytes per element, exceed L2, so every launch streams them from HBM)."""
    from tuckmill_b200 import cuda

    ctx = cuda.CudaContext(device)
    rows, cols = shape.vocab, shape.hidden
    base = T.q8_0_matrix(0, 99, 2048, cols)
    raw = np.tile(base, ((rows + 2047) // 2048, 1, 1))[:rows]
    # Two copies used in turn, as in a real step where the head's weights were evicted from L2 by the
    # layers' before they are read again.
    ws = [ctx.q8_0_matrix(raw, rows, cols) for _ in range(2)]
    x = ctx.floats(T.activations(0, 98, cols))
    y = ctx.buffer(rows * 4)
    st = torch.cuda.ExternalStream(ctx.stream(), device=device)
    n = 20
    ctx.begin_group()  # one replayed graph of n launches: no host gap between them
    for i in range(n):
        ctx.q8_0_gemv(ws[i % 2], x, y, rows, cols)
    graph = ctx.end_group_retain()
    graph.launch()
    ctx.fence()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        e0.record()
    graph.launch()
    with torch.cuda.stream(st):
        e1.record()
    ctx.fence()
    torch.cuda.synchronize()
    graph.free()
    us = e0.elapsed_time(e1) * 1e3 / n
    nbytes = rows * cols + rows * (cols // 32) * 2 + 4 * cols + 4 * rows
    out = {"rows": rows, "cols": cols, "us_per_launch": us, "bytes_per_launch": nbytes,
           "achieved": nbytes / (us * 1e3), "unit": "GB/s", "frac": nbytes / (us * 1e3) / hbm_gbs,
           "traffic": None, "traffic_analytic": nbytes,
           "traffic_note": "measured DRAM traffic of this launch is in the committed ncu summary, not repeated here"}
    for b in ws + [x, y]:
        b.free()
    ctx.close()
    return out


def gemm_rooflines(device, torch):
    """The prefill half of the metric: the tensor-core Q8_0 GEMM alone (tm_cuda_q8_0_gemm_mma: the f16
    copy of X plus the tcgen05 kernel) at the single-operator configuration (3072 x 1024, M = 512)
    and at an 8B-scale projection (12288 x 4096, M = 2048).  CUDA events around one replayed graph of
    n launches that rotate over enough copies of the weights to exceed L2; FLOPs = 2 M N K against the
    measured dense bf16 peak (the stand-in for the f16 tensor peak)."""
    from tuckmill_b200 import cuda

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak, kind = (float(peaks["bf16_tflops"]), "measured") if "bf16_tflops" in peaks else (1590.0, "fallback")
    ctx = cuda.CudaContext(device)
    st = torch.cuda.ExternalStream(ctx.stream(), device=device)
    out = []
    for rows, cols, m in ((3072, 1024, 512), (12288, 4096, 2048)):
        base = T.q8_0_matrix(0, 97, min(rows, 1024), cols)
        raw = np.tile(base, ((rows + base.shape[0] - 1) // base.shape[0], 1, 1))[:rows]
        copies = max(2, int(140e6 // (rows * cols * 1.0625)) + 1)
        ws = [ctx.q8_0_matrix(raw, rows, cols) for _ in range(copies)]
        x = ctx.buffer(m * cols * 4)
        x.upload(0, T.activations(0, 96, m * cols))
        y = ctx.buffer(m * rows * 4)
        ctx.mma_workspace_reserve(cuda.mma_workspace_bytes(cols, m))
        n = max(copies, 12)
        ctx.begin_group()
        for i in range(n):
            ctx.q8_0_gemm_mma(ws[i % copies], x, y, rows, cols, m)
        graph = ctx.end_group_retain()
        for _ in range(3):
            graph.launch()
        ctx.fence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(st):
            e0.record()
        graph.launch()
        with torch.cuda.stream(st):
            e1.record()
        ctx.fence()
        torch.cuda.synchronize()
        graph.free()
        assert not ctx.mma_aborted()
        us = e0.elapsed_time(e1) * 1e3 / n
        tf = 2.0 * m * rows * cols / us / 1e6
        out.append({"bound": "tensor", "rows": rows, "cols": cols, "batch": m, "us_per_launch": us, "achieved": tf,
                    "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                    "kernel": "x_to_f16_kernel + q8_gemm_mma_kernel<%d>" % ctx.mma_last_tile(),
                    "weights": "%d copies in turn (%.0f MB)" % (copies, copies * rows * cols * 1.0625 / 1e6),
                    "peak_source": "MEASURED_PEAKS.json bf16_tflops (%s), burst" % kind})
        for b in ws + [x, y]:
            b.free()
    ctx.close()
    return out


def run_cuda(args):
    import torch
    import torch.distributed as dist

    from tuckmill_b200 import engine as E

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    shape, prompt_n, decode_n = WORKLOADS[args.workload]
    if rank == 0:
        path = artifact(args.workload, args.seed)
    if world > 1:
        dist.barrier()
    path = artifact(args.workload, args.seed)
    context = prompt_n + decode_n + 16
    # 8B-scale projections want wider prefill chunks (the GEMM reaches its rate from M = 2048)
    prefill_batch = 2048 if shape.hidden >= 4096 else 0
    eng = E.Engine(path, context=context, device=local, prefill_batch=prefill_batch)
    stream = torch.cuda.ExternalStream(eng.stream(), device=local)
    prompt = T.token_ids(args.seed + 1000 * rank, prompt_n, shape.vocab)
    hbm_gbs, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        eng.fence()
        torch.cuda.synchronize()

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e.record()
        return e

    # ---- device-resident arm: prefill, then the decode graph replayed ----
    def session():
        eng.reset()
        e0 = ev()
        eng.prefill(prompt, want_token=True)
        e1 = ev()
        eng.decode_steps(decode_n - 1)
        e2 = ev()
        return e0, e1, e2

    for _ in range(args.warmup):
        session()
    barrier()
    launches0 = _launches(eng)
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        evs = [session() for _ in range(args.steps)]
        barrier()
        wall = time.perf_counter() - t0
    launches = _launches(eng) - launches0
    prefill_ms = sum(a.elapsed_time(b) for a, b, c in evs)
    decode_ms = sum(b.elapsed_time(c) for a, b, c in evs)
    total_ms = prefill_ms + decode_ms
    tokens = eng_tokens = None

    # ---- end-to-end arm: the public generate() call with host buffers ----
    for _ in range(max(1, args.warmup // 2)):
        eng.generate(prompt, decode_n)
    barrier()
    spans, ttfts, gen = 0, 0, 0
    for _ in range(args.steps):
        tokens, st = eng.generate(prompt, decode_n)
        spans += st.decode_span_ns
        ttfts += st.ttft_ns
        gen += st.generated - 1
        h2d, d2h = st.h2d_bytes, st.d2h_bytes
    barrier()

    vals = torch.tensor([decode_ms, total_ms, prefill_ms, spans / 1e6, ttfts / 1e6], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    decode_ms, total_ms, prefill_ms, span_ms, ttft_ms = vals.tolist()
    dec_tokens = args.steps * (decode_n - 1)
    value = world * dec_tokens / (decode_ms / 1e3)
    e2e = world * gen / (span_ms / 1e3)

    eng.close()
    # several sequences at once on one GPU (single-process runs; under torchrun the row-split leg carries its own)
    batched = batched_leg(args, E, torch, dist, local, world, path, shape, prompt_n, decode_n,
                          args.sequences) if args.sequences > 1 and world == 1 else None
    split = row_split_leg(args, E, dist, torch, rank, local, world, path, context, shape, prompt_n, decode_n,
                          tokens) if world > 1 else None
    eng = E.Engine(path, context=context, device=local, prefill_batch=prefill_batch) if rank == 0 else None

    if rank == 0:
        roof = gemv_roofline(eng, shape, hbm_gbs, 1e3 * decode_ms / dec_tokens, prompt_n)
        roof["lm_head"] = lm_head_roofline(local, shape, hbm_gbs, torch)
        roof["copy_gbs_this_gpu"] = copy_bandwidth(torch, local)
        roof["lm_head"]["frac_of_this_gpu_copy"] = roof["lm_head"]["achieved"] / roof["copy_gbs_this_gpu"]
        roof["peak_source"] = f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"
        step_bytes = shape.decode_weight_bytes()
        cpu = cpu1 = None
        if not args.no_cpu:
            v, threads, one_core, sample = cpu_leg(args.workload, args.seed, decode_sample=16, one_core_sample=3)
            cpu = {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample}
            cpu1 = {"value": one_core, "unit": "tok/s", "cores": 1, "kind": "port",
                    "sample": "3 further decode steps of the same session on one thread (the reference executor "
                              "is single-threaded)"}
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8 x s8 -> s32 tensor-core products, f32 accumulate",
            "data": "synthetic",
            "config": bench_config(args.workload, args.seed),
            "run": {"prefill_chunk": prefill_batch or 512,
                    "parallelism": f"replicas x{world}" if world > 1 else "single",
                    "l2": "per-token weight stream %.0f MB exceeds the 126 MB L2" % (step_bytes / 1e6)},
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ttft_ms": ttft_ms / args.steps, "prefill_tok_s": world * args.steps * prompt_n / (ttft_ms / 1e3)},
            "gpu_launches": int(launches),
            "roofline": roof,
            "roofline_gemm": gemm_rooflines(local, torch) if args.workload == "qwen3-0.6b" else None,
            "cpu_baseline": cpu,
            "cpu_baseline_1core": cpu1,
            "clocks": clocks.summary(),
            "prefill_tok_s": world * args.steps * prompt_n / (prefill_ms / 1e3),
            "decode_us_per_token": 1e3 * decode_ms / dec_tokens,
            "decode_step_hbm_frac": step_bytes / (1e3 * decode_ms / dec_tokens * 1e3) / hbm_gbs,
            "wall_s": wall,
            "tokens_head": [int(t) for t in tokens[:8]],
        }
        if batched is not None:
            line["batched"] = batched
        if split is not None:
            line["row_split"] = split
        print(json.dumps(line), flush=True)
    if eng is not None:
        eng.close()
    if world > 1:
        dist.destroy_process_group()


def batched_leg(args, E, torch, dist, local, world, path, shape, prompt_n, decode_n, sequences, shard=None):
    """Decode of `sequences` concurrent requests of the workload in ONE recorded step (one row per
    sequence through the batched projections, every sequence attending to its own KV planes): the
    serving shape of the 8-GPU configuration.  Device-timed like `value` (events on the engine's
    stream, max over ranks when the model is split); `e2e_decode_tok_s` goes through
    generate_batch() with host buffers.  With `shard` = (rank, world, comm_id) the ONE model is split
    by output rows and every exchange carries `sequences` rows."""
    context = prompt_n + decode_n + 16
    kw = dict(shard_rank=shard[0], shard_world=shard[1], comm_id=shard[2]) if shard else {}
    eng = E.Engine(path, context=context, device=local, sequences=sequences,
                   prefill_batch=2048 if shape.hidden >= 4096 else 0, **kw)
    stream = torch.cuda.ExternalStream(eng.stream(), device=local)
    prompts = [T.token_ids(args.seed + 7919 * (s + 1), prompt_n, shape.vocab) for s in range(sequences)]

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e.record()
        return e

    def session():
        eng.reset()
        e0 = ev()
        for s in range(sequences):
            eng.prefill_seq(s, prompts[s], want_token=True)
        e1 = ev()
        eng.decode_steps_batch(decode_n - 1)
        e2 = ev()
        return e0, e1, e2

    steps = max(1, min(args.steps, 2))
    session()
    if world > 1 and shard:
        dist.barrier()
    eng.fence()
    l0 = _launches(eng)
    evs = [session() for _ in range(steps)]
    eng.fence()
    torch.cuda.synchronize()
    launches = _launches(eng) - l0
    toks, st = eng.generate_batch(prompts, decode_n)
    vals = torch.tensor([sum(a.elapsed_time(b) for a, b, c in evs), sum(b.elapsed_time(c) for a, b, c in evs),
                         st.decode_span_ns / 1e6], dtype=torch.float64, device="cuda")
    if world > 1 and shard:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms, span_ms = vals.tolist()
    n_steps = steps * (decode_n - 1)
    info = eng.refresh_info()
    # bytes one step must read: the weights once, and every sequence's K and V rows up to its position
    kv_row = 2 * shape.layers * shape.kv_heads * shape.head_dim * 2
    window = shape.window if shape.arch == "gemma3" and shape.window else 0
    mean_pos = prompt_n + decode_n / 2
    kv_read = sequences * kv_row * (mean_pos if not window else min(mean_pos, window))  # upper bound for Gemma's global layers
    share = (shard[1] if shard else 1)
    step_bytes = (shape.decode_weight_bytes() + kv_read) / share
    hbm_gbs, _ = measured_peaks()
    us_step = 1e3 * decode_ms / n_steps
    out = {
        "sequences": sequences, "prompt_tokens": prompt_n, "decode_tokens": decode_n,
        "parallelism": f"one model split x{shard[1]}" if shard else "single",
        "decode_tok_s": sequences * n_steps / (decode_ms / 1e3),
        "us_per_step": us_step,
        "prefill_tok_s": steps * sequences * prompt_n / (prefill_ms / 1e3),
        "e2e_decode_tok_s": (st.generated - sequences) / (span_ms / 1e3),
        "h2d_bytes_per_step": int(st.h2d_bytes), "d2h_bytes_per_step": int(st.d2h_bytes),
        "gpu_launches": int(launches),
        "step_bytes_per_gpu": int(step_bytes),
        "step_hbm_frac": step_bytes / (us_step * 1e3) / hbm_gbs,
        "kv_bytes_per_gpu": int(info.plan_state),
        "tokens_head": [int(t[1]) if len(t) > 1 else -1 for t in toks[:8]],
    }
    eng.close()
    return out


def row_split_leg(args, E, dist, torch, rank, local, world, path, context, shape, prompt_n, decode_n, replica_tokens):
    """The same session with ONE model split over all ranks (each rank holds 1/world of
    every projection, of the head and of the KV cache: q|k|v, gate|up and the head by
    output rows, o and down by input columns; two exchanges per layer inside the
    replayed decode graph, pushed through peer memory).  Strong scaling of a single
    sequence: reported beside the replica figure, not as `value`."""
    if os.environ.get("TM_BENCH_ROW_SPLIT", "1") == "0":
        return {"unavailable": "switched off by TM_BENCH_ROW_SPLIT=0"}
    try:
        from tuckmill_b200 import sharding as S
        S.shard_geometry(shape, world)
    except ValueError as e:
        return {"unavailable": str(e)}
    def fresh_comm_id() -> bytes:  # one communicator per engine: an id is not reused
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident.copy_(torch.frombuffer(bytearray(E.comm_id()), dtype=torch.uint8))
        dist.broadcast(ident, 0)
        return bytes(ident.cpu().numpy().tobytes())

    eng = E.Engine(path, context=context, device=local, shard_rank=rank, shard_world=world,
                   comm_id=fresh_comm_id(), prefill_batch=2048 if shape.hidden >= 4096 else 0)
    stream = torch.cuda.ExternalStream(eng.stream(), device=local)
    prompt = T.token_ids(args.seed, prompt_n, shape.vocab)  # rank 0's prompt of the replica arm, on every rank

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e.record()
        return e

    def session():
        eng.reset()
        e0 = ev()
        eng.prefill(prompt, want_token=True)
        e1 = ev()
        eng.decode_steps(decode_n - 1)
        e2 = ev()
        return e0, e1, e2

    for _ in range(args.warmup):
        session()
    dist.barrier()
    eng.fence()
    evs = [session() for _ in range(args.steps)]
    eng.fence()
    torch.cuda.synchronize()
    tokens, st = eng.generate(prompt, decode_n)
    vals = torch.tensor([sum(a.elapsed_time(b) for a, b, c in evs), sum(b.elapsed_time(c) for a, b, c in evs),
                         st.decode_span_ns / 1e6], dtype=torch.float64, device="cuda")
    dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms, span_ms = vals.tolist()
    info = eng.refresh_info()
    # where a split step's time goes: every operator dispatched on its own with events around it (all ranks
    # make the same calls; rank 0's table is printed)
    eng.reset()
    eng.prefill(prompt, want_token=True)
    eng.decode_ungrouped(2)
    eng.fence()
    eng.profile(True)
    eng.decode_ungrouped(4)
    eng.fence()
    by_op = {n: round(ns / 4 / 1e3, 2) for n, ns, c in sorted(eng.profile_rows())}
    eng.profile(False)
    out = {
        "by_operator_us_per_step_ungrouped": by_op,
        "parallelism": f"one model split x{world} (q|k|v, gate|up, head by output rows; o, down by input columns; "
                       "two exchanges per layer pushed through peer memory on the compute stream)", "scaling": "strong",
        "decode_tok_s": args.steps * (decode_n - 1) / (decode_ms / 1e3),
        "decode_us_per_token": 1e3 * decode_ms / (args.steps * (decode_n - 1)),
        "prefill_tok_s": args.steps * prompt_n / (prefill_ms / 1e3),
        "e2e_decode_tok_s": (st.generated - 1) / (span_ms / 1e3),
        "per_rank_weight_bytes": int(info.plan_weights), "per_rank_kv_bytes": int(info.plan_state),
        "tokens_equal_single_device": bool(replica_tokens is not None and list(tokens) == list(replica_tokens)),
        # The column-split projections add their partial sums in rank order, not in the single-device order:
        # the streams may part at a near-tie (tolerance mode); how long they agree is reported beside the flag.
        "tokens_common_prefix": (None if replica_tokens is None else
                                 next((i for i, (a, b) in enumerate(zip(tokens, replica_tokens)) if a != b),
                                      min(len(tokens), len(replica_tokens)))),
    }
    eng.close()
    if args.sequences > 1:
        out["batched"] = batched_leg(args, E, torch, dist, local, world, path, shape, prompt_n, decode_n, args.sequences,
                                     shard=(rank, world, fresh_comm_id()))
    return out


SWEEP_SHAPES = [(4096, 4096), (12288, 4096), (4096, 12288), (151936, 4096)]
SWEEP_BATCHES = [1, 8, 32, 128, 512, 2048, 8192]


def run_sweep(args):
    """The Q8_0 projection sweep at Qwen3-8B shapes, split by output rows over the
    ranks: every rank multiplies its N/G rows with the single-device kernel (GEMV at
    M = 1, the bit-identical batched form up to 8, the tensor-core GEMM above) and an
    all-gather reassembles Y -- once as ncclAllGather (+ interleave), once as a push
    through peer memory.  Per case: device time of the multiply alone, of each
    exchange alone, and of multiply + exchange back to back (each a replayed graph,
    CUDA events, max over ranks).  Rank 0 prints one JSON line; a profiling aid, not `value`."""
    import torch
    import torch.distributed as dist

    from tuckmill_b200 import cuda

    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = cuda.CudaContext(local)
    if world > 1:
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident.copy_(torch.frombuffer(bytearray(cuda.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(ident, 0)
        ctx.comm_init(bytes(ident.cpu().numpy().tobytes()), rank, world)
    st = torch.cuda.ExternalStream(ctx.stream(), device=local)
    hbm_gbs, _ = measured_peaks()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))

    def timed(record, reps):
        ctx.begin_group()
        for _ in range(reps):
            record()
        g = ctx.end_group_retain()
        g.launch()
        ctx.fence()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(st):
            e0.record()
        g.launch()
        with torch.cuda.stream(st):
            e1.record()
        ctx.fence()
        torch.cuda.synchronize()
        g.free()
        v = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    cases = []
    for rows, cols in SWEEP_SHAPES:
        local_rows = rows // world
        base = T.q8_0_matrix(args.seed, 1, min(local_rows, 1024), cols)
        copies = 2 if local_rows * cols < 200e6 else 1  # small slices alternate so they are not L2-resident
        ws = [ctx.q8_0_matrix(np.tile(base, ((local_rows + base.shape[0] - 1) // base.shape[0], 1, 1))[:local_rows],
                              local_rows, cols) for _ in range(copies)]
        for m in SWEEP_BATCHES:
            if m * rows * 4 > 3 << 30:
                continue  # a gathered Y above 3 GiB is left out
            x = ctx.buffer(m * cols * 4)
            x.upload(0, T.activations(args.seed, 2, min(m * cols, 1 << 22)))
            y_loc = ctx.buffer(m * local_rows * 4)
            y = ctx.buffer(m * rows * 4) if world > 1 else y_loc
            stage = ctx.buffer(m * rows * 4) if world > 1 and m > 1 else y
            if m > 8:
                ctx.mma_workspace_reserve(cuda.mma_workspace_bytes(cols, m))
            turn = [0]

            def multiply():
                w = ws[turn[0] % copies]
                turn[0] += 1
                if m == 1:
                    ctx.q8_0_gemv(w, x, y_loc, local_rows, cols)
                elif m <= 8:
                    ctx.q8_0_gemm(w, x, y_loc, local_rows, cols, m)
                else:
                    ctx.q8_0_gemm_mma(w, x, y_loc, local_rows, cols, m)

            def gather():
                ctx.all_gather_rows_f32(y_loc, stage, y, m, local_rows)

            def both():
                multiply()
                gather()

            # the same exchange as a push through peer memory (two target views used in turn)
            arena = ctx.symm_buffer(2 * m * rows * 4) if world > 1 else None
            views = [arena.view(i * m * rows * 4, m * rows * 4) for i in range(2)] if world > 1 else []
            pturn = [0]

            def push():
                ctx.push_rows_f32(y_loc, views[pturn[0] % 2], m, local_rows)
                pturn[0] += 1

            def both_push():
                multiply()
                push()

            reps = 20 if m * rows * cols < 2e11 else 4
            t_mul = timed(multiply, reps)
            t_ag = timed(gather, reps) if world > 1 else 0.0
            t_both = timed(both, reps) if world > 1 else t_mul
            t_push = timed(push, reps) if world > 1 else 0.0
            t_both_push = timed(both_push, reps) if world > 1 else t_mul
            nbytes = rows * (cols // 32) * 34 + 4 * m * cols * world + 4 * m * rows
            case = {"rows": rows, "cols": cols, "batch": m, "us_multiply": round(t_mul, 2),
                    "us_all_gather": round(t_ag, 2), "us_both": round(t_both, 2),
                    "us_push": round(t_push, 2), "us_both_push": round(t_both_push, 2),
                    "tflops": round(2.0 * m * rows * cols / t_both / 1e6, 1),
                    "gbs": round(nbytes / t_both / 1e3, 1)}
            case["frac"] = round(case["gbs"] / (hbm_gbs * world), 3) if m <= 8 else round(case["tflops"] / (tf_peak * world), 3)
            case["bound"] = "hbm" if m <= 8 else "tensor"
            cases.append(case)
            for b in views:
                b.free()
            for b in {id(b): b for b in (x, y_loc, y, stage)}.values():
                b.free()
            if arena is not None:
                assert ctx.symm_status(arena) == 0, "a peer-memory wait ran out"
                arena.free()
        for w in ws:
            w.free()
    if rank == 0:
        print(json.dumps({"workload": "q8_0 projection sweep, output rows split over the ranks", "n_gpus": world,
                          "peaks": {"hbm_gbs": hbm_gbs, "tflops": tf_peak, "per": "GPU; frac is of n_gpus x peak"},
                          "cases": cases}), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_op(args):
    """Small fixed cases for profiler captures (`--op`): a few launches of one
    kernel at a stated shape, or one prefill plus three decode steps of the
    workload.  Prints what ran; no JSON line, not a measurement."""
    from tuckmill_b200 import cuda, engine as E

    if args.op == "slice":
        shape, prompt_n, decode_n = WORKLOADS[args.workload]
        eng = E.Engine(artifact(args.workload, args.seed), context=prompt_n + decode_n + 16)
        for _ in range(2):
            eng.reset()
            eng.prefill(T.token_ids(args.seed, prompt_n, shape.vocab), want_token=True)
            eng.decode_steps(3)
            eng.fence()
        print("slice: 2 x (prefill %d + 3 decode steps), %d launches" % (prompt_n, _launches(eng)))
        eng.close()
        return
    ctx = cuda.CudaContext(0)
    if args.op == "attn":
        # decode attention of `--sequences` sequences at position `--batch`, geometry of the workload
        shape = WORKLOADS[args.workload][0]
        S, pos, heads, kvh, hd = args.sequences, args.batch, shape.heads, shape.kv_heads, shape.head_dim
        cap = pos + 64
        plane = kvh * cap * hd
        rng = np.random.default_rng(0)
        fill = (rng.standard_normal(min(S * plane, 1 << 24)) * 0.5).astype(np.float16)
        caches = []
        for _ in range(2):
            kc = ctx.buffer(S * plane * 2)
            for off in range(0, S * plane, fill.size):
                kc.upload(off * 2, fill[:min(fill.size, S * plane - off)])
            caches.append(kc)
        one = ctx.floats(np.ones(hd, np.float32))
        inv = ctx.floats((shape.rope_base ** (-np.arange(hd // 2, dtype=np.float64) * 2 / hd)).astype(np.float32))
        q = ctx.floats(T.activations(0, 1, S * heads * hd))
        k, v = ctx.floats(T.activations(0, 2, S * kvh * hd)), ctx.floats(T.activations(0, 3, S * kvh * hd))
        out = ctx.buffer(S * heads * hd * 4)
        sb = ctx.buffer(S * cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
        sb.zero()
        pb, st = ctx.from_array(np.full(S, pos, np.uint32)), ctx.buffer(4, shared=True)
        st.zero()
        for _ in range(3):
            ctx.attention_decode_batch(q, k, v, one, one, inv, caches[0], caches[1], out, sb, pb, st, S, heads, kvh, hd, hd,
                                       cap, 0, shape.eps, float(1 / np.sqrt(hd)), False)
        ctx.fence()
        print("attn %s: %d sequences at position %d, 3 launches, %.1f MB of K and V per launch" %
              (args.workload, S, pos, S * 2 * kvh * (pos + 1) * hd * 2 / 1e6))
        return
    rows, cols, m = args.rows, args.cols, args.batch
    base = T.q8_0_matrix(0, 1, min(rows, 1024), cols)
    w = ctx.q8_0_matrix(np.tile(base, ((rows + base.shape[0] - 1) // base.shape[0], 1, 1))[:rows], rows, cols)
    x = ctx.buffer(m * cols * 4)
    x.upload(0, T.activations(0, 2, min(m * cols, 1 << 22)))
    y = ctx.buffer(m * rows * 4)
    for _ in range(3):
        if args.op == "gemm":
            ctx.q8_0_gemm_mma(w, x, y, rows, cols, m)
        else:
            ctx.q8_0_gemv(w, x, y, rows, cols)
    ctx.fence()
    print("%s %dx%d batch %d: 3 launches, aborted=%s" % (args.op, rows, cols, m, ctx.mma_aborted()))


def _launches(eng) -> int:
    from tuckmill_b200 import cuda as C

    return int(C.load_library().tm_cuda_kernel_launches(eng.cuda_ctx()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="qwen3-0.6b", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--sequences", type=int, default=32,
                    help="concurrent sequences of the batched-decode leg reported beside the one-sequence metric "
                         "(1 switches the leg off)")
    ap.add_argument("--op", choices=["gemv", "gemm", "slice", "sweep", "attn"],
                    help="profiler case / projection sweep instead of the benchmark")
    ap.add_argument("--rows", type=int, default=12288)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=2048)
    args = ap.parse_args()
    if args.op == "sweep":
        run_sweep(args)
    elif args.op:
        run_op(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
