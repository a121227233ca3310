#!/usr/bin/env python
"""Benchmark of the batched sampler hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the sampler over one batch of synthetic logits.  The
default workload is the headline shape: 256 rows x vocab 201088 fp32 logits
with the config-1 parameters (T=0.7, top_k=50, top_p=0.9, min_p=0.05), rows
drawn as 3*N(0,1) plus 32 boosted entries and forced duplicates.  With N > 1
(launched by torch.distributed.run) every rank samples its own 256 rows — rows
are independent, so there is no data-path collective (weak scaling) — and the
two sharded workloads of the benchmark configurations are timed as well.

One JSON line is printed by rank 0:
  value      rows/s with logits and parameters resident in HBM: a CUDA graph of
             consecutive steps replayed until the timed region is at least half
             a second long (CUDA events, max over ranks).  Consecutive steps are
             independent batches and their launches overlap.
  roofline   achieved HBM GB/s of the streaming kernel (one logits read per row)
             against the measured copy bandwidth of this pool's B200s: `frac`
             for the overlapped launches, `frac_single_launch` for the same
             graph with every launch strictly after the previous one
  e2e        rows/s through moe_sample_batch_host: pinned host logits in, host
             results out, copies inside the timed region; `e2e_device_logits`
             is the same call pattern with the logits left on the device
             (moe_sample_tokens: only 16 bytes per row return to the host)
  cpu_baseline  the reference's own CPU sampler timed on this box's host cores
             on a bounded sample of the same workload (N=1 only)
  config.workloads  (N=1) the other benchmark configurations: time, roofline
             fraction and full-size agreement of the token ids with the CPU oracle
  config.sharded    (N>1) config 4 split by rows and config 5a split by vocabulary

`--impl reference` times only that CPU sampler (all host threads) and prints
the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import __graft_entry__ as graft  # noqa: E402

METRIC = "sampled rows/s at vocab 201088, batch 256"
UNIT = "rows/s"
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only when MEASURED_PEAKS.json is absent
MIN_TIMED_SECONDS = 0.5
GROUP_TIMEOUT = datetime.timedelta(seconds=240)  # process-group watchdog: longer than any rank's host-side work

WORKLOADS = {
    # name: (generator, kwargs, dtype label, description)
    "headline": ("config1_row", dict(rows=256, vocab=201088, dtype="f32"), "f32",
                 "256 rows x vocab 201088 fp32, T=0.7 top_k=50 top_p=0.9 min_p=0.05 (config-1 parameters tiled to batch 256)"),
    "headline_bf16": ("config1_row", dict(rows=256, vocab=201088, dtype="bf16"), "bf16",
                      "256 rows x vocab 201088 bf16, T=0.7 top_k=50 top_p=0.9 min_p=0.05"),
    "config2": ("config2_greedy_temperature", dict(rows=256, vocab=129280), "bf16", "256 rows x vocab 129280 bf16, greedy / T=1 untruncated alternating"),
    "config3": ("config3_mixed", dict(rows=1024, vocab=151936), "f32", "1024 rows x vocab 151936 fp32, mixed per-row parameters"),
    "config4": ("config4_heavy_tail", dict(rows=8192, vocab=201088), "bf16", "8192 rows x vocab 201088 bf16 Student-t(3), top_p=0.95 only"),
    "config5a": ("config5a_large_vocab", dict(rows=64, vocab=1048576), "f32", "64 rows x vocab 1048576 fp32, top_k=64 top_p=0.9 (single GPU)"),
}
# distinct rows generated on the host for config 4; the timed batch tiles them (the generator
# needs about 8 ms per row, and the timing only depends on the distribution of the values)
CONFIG4_DISTINCT_ROWS = 512


def log(*args):
    print(*args, file=sys.stderr, flush=True)


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


def captured_traffic(workload: str):
    """dram bytes per launch of the streaming kernel from the committed ncu summary, or (None, reason)."""
    path = ROOT / "profiles" / "traffic.json"
    try:
        entry = json.loads(path.read_text())[workload]
        return int(entry["dram_bytes_per_launch"]), f"profiles/traffic.json ({entry.get('source', 'ncu capture')})"
    except Exception:
        return None, "no ncu capture of this workload under profiles/"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index = index
        self.period = period_s
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception as error:  # NVML missing: clocks stay unknown
            log("clock sampling unavailable:", error)
            self._nvml = None

    def _reason_names(self, mask: int):
        n = self._nvml
        table = [
            ("hw_slowdown", getattr(n, "nvmlClocksEventReasonHwSlowdown", getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8))),
            ("hw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40))),
            ("sw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20))),
            ("sw_power_cap", getattr(n, "nvmlClocksEventReasonSwPowerCap", getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4))),
        ]
        return [name for name, bit in table if mask & bit]

    def _run(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                self.reasons.update(self._reason_names(int(mask)))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._nvml is None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self, where: str):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0, "sampled": where}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "sampled": where}


def host_thread_count() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def bind_to_gpu_numa_node(local_rank: int):
    """Restricts this process to the CPUs of the NUMA node its GPU hangs on, so that the page-locked
    staging buffers it allocates afterwards live next to the GPU.  Returns a description."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        bus_id = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus_id = (bus_id.decode() if isinstance(bus_id, bytes) else bus_id).lower()
        if len(bus_id.split(":")[0]) == 8:
            bus_id = bus_id[4:]
        node = int(Path(f"/sys/bus/pci/devices/{bus_id}/numa_node").read_text().strip())
        if node < 0:
            return "no NUMA information for the GPU"
        cpulist = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
        cpus = set()
        for part in cpulist.split(","):
            low, _, high = part.partition("-")
            cpus.update(range(int(low), int(high or low) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return f"GPU on NUMA node {node}, none of its CPUs available to this process"
        os.sched_setaffinity(0, allowed)
        return f"bound to NUMA node {node} ({len(allowed)} CPUs)"
    except Exception as error:
        return f"not bound ({type(error).__name__})"


def generate(package, workloads, name, rank=0, rows=None):
    generator, kwargs, dtype_label, description = WORKLOADS[name]
    function = getattr(workloads, generator)
    kwargs = dict(kwargs)
    if rows is not None:
        kwargs["rows"] = rows
    if generator in ("config1_row", "config4_heavy_tail"):
        kwargs["row_offset"] = rank * kwargs["rows"]
    return function(package.ROW_PARAMS_DTYPE, **kwargs), dtype_label, description


def workload_config(name, world, sharding=None):
    """The keys both arms (this library and --impl reference) report for a workload."""
    _, kwargs, _, description = WORKLOADS[name]
    return {"workload": description, "rows_per_gpu": kwargs["rows"], "vocab": kwargs["vocab"],
            "sharding": sharding or ("rows" if world > 1 else "none")}


def cpu_sampler_rate(oracle, logits, params, uniforms, rows_sample, threads):
    sample = slice(0, rows_sample)
    start = time.perf_counter()
    result = oracle.sample_batch(logits[sample], params["temperature"][sample], params["top_k"][sample], params["top_p"][sample],
                                 params["min_p"][sample], uniforms[sample], threads=threads)
    elapsed = time.perf_counter() - start
    return rows_sample / elapsed, elapsed, result


def run_reference_arm(args):
    """The reference's own CPU sampler on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0  # only rank 0 measures the CPU arm
    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    from oracle import oracle as oracle_module
    oracle = oracle_module.best()
    threads = host_thread_count()
    (logits, params), dtype_label, _ = generate(package, workloads, args.workload, rows=min(WORKLOADS[args.workload][1]["rows"], 512))
    rows = logits.shape[0]
    uniforms = np.array([oracle_module.port().philox_uniform(p["seed"], p["row_id"], p["step"]) for p in params], dtype=np.float32)
    # size a step so that warmup + steps end within about a minute of wall clock
    probe_rows = min(rows, max(threads, 8))
    rate, _, _ = cpu_sampler_rate(oracle, logits, params, uniforms, probe_rows, threads)
    budget_s = 60.0
    rows_per_step = int(max(1, min(rows, rate * budget_s / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        cpu_sampler_rate(oracle, logits, params, uniforms, rows_per_step, threads)
    start = time.perf_counter()
    for _ in range(args.steps):
        cpu_sampler_rate(oracle, logits, params, uniforms, rows_per_step, threads)
    elapsed = time.perf_counter() - start
    value = rows_per_step * args.steps / elapsed
    sample = f"{rows_per_step} of {WORKLOADS[args.workload][1]['rows']} rows per step, {args.steps} steps, {threads} host threads over independent rows"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_label,
        "data": "synthetic", "config": workload_config(args.workload, args.gpus),
        "run": {"rows_per_step": rows_per_step},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": oracle.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---- timing helpers -----------------------------------------------------------------


def to_device(torch, array):
    if array.dtype == np.uint16:
        return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(array).cuda()


def time_step_graph(torch, step, steps, chunk, min_seconds, clocks=None, barrier=None):
    """Captures `chunk` consecutive calls of step(i) in one CUDA graph and replays it until at least
    `steps` steps and `min_seconds` have been timed.  Returns (ms per step, timed steps, replays)."""
    chunk = max(1, min(chunk, steps))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(chunk):
            step(i)
    graph.replay()
    torch.cuda.synchronize()
    # a short probe sizes the timed region
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(3):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    per_replay_s = max(start.elapsed_time(stop) / 3 * 1e-3, 1e-7)
    replays = max((steps + chunk - 1) // chunk, int(np.ceil(min_seconds / per_replay_s)))
    if barrier is not None:
        # every rank must replay the same number of times: the graph may hold a collective, and the
        # probe above times differently on every rank
        parallel = __import__(graft.PACKAGE_NAME + ".parallel", fromlist=["parallel"])
        replays = parallel.agree_on_maximum(replays, device="cuda")
        barrier()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.start()
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.stop()
    if barrier is not None:
        barrier()
    elapsed_ms = start.elapsed_time(stop)
    return elapsed_ms / (replays * chunk), replays * chunk, replays, graph


def fresh_outputs(torch, rows):
    return {"token": torch.empty(rows, dtype=torch.int32, device="cuda"), "probability": torch.empty(rows, dtype=torch.float32, device="cuda"),
            "flags": torch.empty(rows, dtype=torch.int32, device="cuda"), "status": torch.empty(rows, dtype=torch.int32, device="cuda"), "topk": None}


def oracle_tokens(oracle, package, logits, params, step_offset, rows, threads):
    uniforms = np.array([package.philox_uniform(p["seed"], p["row_id"], int(p["step"]) + step_offset) for p in params[:rows]], dtype=np.float32)
    return oracle.sample_batch(logits[:rows], params["temperature"][:rows], params["top_k"][:rows], params["top_p"][:rows],
                               params["min_p"][:rows], uniforms, threads=threads)


def time_sampler_workload(torch, package, sampler, batches, params, steps, min_seconds, chunk=32):
    """Overlapped and strictly serial graph replays of one resident workload; returns a dict."""
    rotation = len(batches)
    out = sampler.sample_batch(batches[0], params)
    torch.cuda.synchronize()

    def step(i):
        sampler.sample_batch(batches[i % rotation], None, step_offset=i, out=out)

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    result = {}
    for label, overlap in (("overlapped", True), ("single_launch", False)):
        sampler.set_overlap(overlap)
        ms, timed, replays, graph = time_step_graph(torch, step, steps, chunk, min_seconds)
        result[label] = {"ms_per_step": ms, "timed_steps": timed}
        del graph
    sampler.set_overlap(False)
    return result


# ---- the other benchmark configurations (one GPU) ------------------------------------


def run_router_bench(args, as_dict=False):
    """Config 5b: router Top-8 with sigmoid scoring over 4096 tokens x 256 experts (one GPU).

    Latency-bound (4 MiB in, 32768 routes out): reported as time and tokens/s, not as a roofline fraction."""
    import torch
    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    torch.cuda.set_device(0)
    tokens, experts, top_k = 4096, 256, 8
    logits_host, bias_host = workloads.config5b_router(tokens, experts)
    sampler = package.Sampler(max_rows=1, max_vocab=1)
    logits = [torch.from_numpy(np.roll(logits_host, shift, axis=0)).cuda() for shift in range(4)]
    bias = torch.from_numpy(bias_host).cuda()
    plan = sampler.router_dispatch(logits[0], top_k, score_function=package.ROUTER_SIGMOID, selection_bias=bias)
    hidden = torch.randn(tokens, 4096, device="cuda")
    torch.cuda.synchronize()

    def step(i):
        sampler.router_dispatch(logits[i % 4], top_k, score_function=package.ROUTER_SIGMOID, selection_bias=bias, out=plan)

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    ms, timed, replays, graph = time_step_graph(torch, step, min(args.steps, 256), 32, 0.1)
    del graph
    # regroup gather of the routed hidden rows (hidden size 4096 fp32): HBM-bound copy
    gathered = sampler.regroup_gather(hidden, plan.route_token)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(50):
        sampler.regroup_gather(hidden, plan.route_token)
    stop.record()
    torch.cuda.synchronize()
    gather_ms = start.elapsed_time(stop) / 50
    gather_bytes = 2 * gathered.numel() * 4
    # reference dispatcher on the host cores
    from oracle import oracle as oracle_module
    oracle = oracle_module.best()
    t0 = time.perf_counter()
    want = oracle.expert_dispatch(logits_host, tokens, experts, top_k, score_function=1, selection_bias=bias_host)
    cpu_s = time.perf_counter() - t0
    step(0)
    torch.cuda.synchronize()
    got_tokens = plan.route_token.cpu().numpy().view(np.uint32)
    got_ranks = plan.route_rank.cpu().numpy().view(np.uint32)
    equal = bool(got_tokens.size == want["token"].size and np.array_equal(got_tokens, want["token"]) and np.array_equal(got_ranks, want["rank"]))
    peak, _ = measured_peak()
    line = {"metric": "router tokens/s, stable Top-8 of 256 experts, sigmoid scoring, 4096 tokens", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": timed, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 5b: 4096 tokens x 256 experts fp32 N(0,1) + bias N(0,0.1), sigmoid, top_k 8, renormalised", "kernels_per_step": 3},
            "gpu_launches": 3 * timed,
            "regroup_gather": {"ms": gather_ms, "achieved_gbs": gather_bytes / (gather_ms * 1e-3) / 1e9, "peak_gbs": peak, "frac": gather_bytes / (gather_ms * 1e-3) / 1e9 / peak,
                               "shape": "32768 routes x 4096 fp32 columns",
                               "note": "algorithmic bytes = one read and one write per routed row; the 64 MiB of hidden rows are each read top_k times "
                                       "and stay in L2, so DRAM sees about (1 + 1/top_k) / 2 of these bytes and the fraction can exceed 1"},
            "cpu_baseline": {"value": tokens / cpu_s, "unit": "tokens/s", "cores": 1, "kind": oracle.kind, "sample": "the whole 4096-token call, single thread (the reference dispatcher is single-threaded)"},
            "routes_equal_to_reference": equal}
    sampler.close()
    if as_dict:
        return line
    print(json.dumps(line), flush=True)
    return 0


def run_speculative_bench(args, as_dict=False):
    """Speculative-decoding verification (session.cpp:776-880): 4 proposed tokens per step against
    5 target and 4 draft rows of vocab 201088 fp32, T=1 / top_k 40 / top_p 0.95.  Three kernels and a
    40-byte upload per step: latency-bound, reported as time per verification."""
    import torch
    package = graft.load_package()
    torch.cuda.set_device(0)
    from oracle import oracle as oracle_module
    oracle = oracle_module.best()
    vocab, draft_count = 201088, 4
    options = (1.0, 40, 0.95, 0.0)
    rng = np.random.default_rng(31)
    cases = []
    for case in range(4):
        target = (2.5 * rng.standard_normal((draft_count + 1, vocab))).astype(np.float32)
        draft = (target[:draft_count] + [0.05, 0.3, 0.6, 1.2][case] * rng.standard_normal((draft_count, vocab)).astype(np.float32)).astype(np.float32)
        proposed = np.array([oracle.sample(draft[j], float(rng.random()), *options)[1] for j in range(draft_count)], dtype=np.int32)
        cases.append((target, draft, proposed))
    device_cases = [(torch.from_numpy(t).cuda(), torch.from_numpy(d).cuda(), torch.from_numpy(p).cuda()) for t, d, p in cases]
    params = np.zeros(1, dtype=package.ROW_PARAMS_DTYPE)
    params["temperature"], params["top_k"], params["top_p"], params["min_p"] = options
    params["seed"], params["row_id"] = 9, 0
    sampler = package.Sampler(max_rows=2 * draft_count + 1, max_vocab=vocab)
    # parity of every case first (also the warm-up)
    equal = 0
    t_cpu = 0.0
    for index, ((target, draft, proposed), device) in enumerate(zip(cases, device_cases)):
        params["step"] = 7 * index
        got = sampler.speculative_verify(device[0], device[1], device[2], params)
        uniforms = np.array([package.philox_uniform(9, 0, 7 * index + i) for i in range(draft_count + 2)], dtype=np.float32)
        t0 = time.perf_counter()
        want = oracle.speculative_verify(target, draft, proposed, uniforms, *options)
        t_cpu += time.perf_counter() - t0
        equal += int(got["status"] == want["status"] == 0 and got["accepted"] == want["accepted"] and got["next_token"] == want["next_token"]
                     and got["uniforms_used"] == want["uniforms_used"])
    out = None
    for i in range(max(args.warmup, 3)):
        out = sampler.speculative_verify(*device_cases[i % 4], params, out=out, sync=False)
    torch.cuda.synchronize()
    steps = min(args.steps, 256)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        sampler.speculative_verify(*device_cases[i % 4], params, out=out, sync=False)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    sampler.close()
    # the scheduler's batch: 32 Sessions verified by one call (the 4 cases repeated, each Session with its own counters)
    sessions = 32
    batch_params = np.repeat(params, sessions)
    batch_params["row_id"] = np.arange(sessions)
    batch_target = torch.stack([device_cases[b % 4][0] for b in range(sessions)])
    batch_draft = torch.stack([device_cases[b % 4][1] for b in range(sessions)])
    batch_proposed = torch.stack([device_cases[b % 4][2] for b in range(sessions)])
    sampler = package.Sampler(max_rows=sessions * (2 * draft_count + 1), max_vocab=vocab)
    records, _ = sampler.speculative_verify_batch(batch_target, batch_draft, batch_proposed, batch_params)
    batch_equal = 0
    for b in range(sessions):
        uniforms = np.array([package.philox_uniform(9, b, int(params["step"][0]) + i) for i in range(draft_count + 2)], dtype=np.float32)
        want = oracle.speculative_verify(*cases[b % 4], uniforms, *options)
        batch_equal += int(records[b]["status"] == want["status"] == 0 and records[b]["accepted"] == want["accepted"]
                           and records[b]["next_token"] == want["next_token"] and records[b]["uniforms_used"] == want["uniforms_used"])
    batch_out = None
    for i in range(3):
        batch_out = sampler.speculative_verify_batch(batch_target, batch_draft, batch_proposed, batch_params, out=batch_out, sync=False)
    torch.cuda.synchronize()
    batch_steps = min(args.steps, 64)
    start.record()
    for i in range(batch_steps):
        sampler.speculative_verify_batch(batch_target, batch_draft, batch_proposed, batch_params, out=batch_out, sync=False)
    stop.record()
    torch.cuda.synchronize()
    batch_ms = start.elapsed_time(stop) / batch_steps
    batch_bytes = sessions * 9 * vocab * 4
    line = {"metric": "speculative verifications/s, 4 proposed tokens, vocab 201088", "value": 1e3 / ms, "unit": "verifications/s", "n_gpus": 1,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "5 target + 4 draft rows x 201088 fp32 2.5*N(0,1) (draft = target + noise), T=1 top_k=40 top_p=0.95; direct C-ABI calls, "
                                   "device-resident logits, 4 cases rotated", "kernels_per_step": 3, "bytes_read_per_step": 9 * vocab * 4},
            "gpu_launches": 3 * steps,
            "cpu_baseline": {"value": len(cases) / t_cpu, "unit": "verifications/s", "cores": 1, "kind": oracle.kind,
                             "sample": f"{len(cases)} verifications, single thread (a Session verifies on its own thread)"},
            "results_equal_to_reference": f"{equal}/{len(cases)}",
            "batched": {"sessions_per_call": sessions, "ms_per_call": batch_ms, "verifications_per_s": sessions * 1e3 / batch_ms,
                        "logits_GBps": batch_bytes / batch_ms / 1e6, "kernels_per_call": 3, "steps": batch_steps,
                        "results_equal_to_reference": f"{batch_equal}/{sessions}"}}
    sampler.close()
    if as_dict:
        return line
    print(json.dumps(line), flush=True)
    return 0


def side_workload(torch, package, workloads, oracle, name, steps, peak, threads):
    """Times one of the other sampler configurations on this GPU and checks the token ids of the
    whole batch (config 4: of its distinct rows) against the CPU oracle."""
    if name == "config4":
        (logits, params), dtype_label, description = generate(package, workloads, name, rows=CONFIG4_DISTINCT_ROWS)
        timed_rows = 2048
    else:
        (logits, params), dtype_label, description = generate(package, workloads, name)
        timed_rows = logits.shape[0]
    rows, vocab = logits.shape
    element = logits.itemsize
    sampler = package.Sampler(max_rows=timed_rows, max_vocab=vocab)
    device = to_device(torch, logits)
    check = sampler.sample_batch(device, params)
    torch.cuda.synchronize()
    want = oracle_tokens(oracle, package, logits, params, 0, rows, threads)
    got = check["token"].cpu().numpy()
    agree = int(np.sum(got == want["token"]))
    if timed_rows != rows:
        repeat = timed_rows // rows
        device = device.repeat(repeat, 1)
        params = np.tile(params, repeat)
        params["row_id"] = np.arange(timed_rows, dtype=np.uint64)
    bytes_per_step = timed_rows * vocab * element
    rotation = 4 if bytes_per_step * 4 <= 8 << 30 else 2
    batches = [device] + [device.roll(shift, 0).contiguous() for shift in range(1, rotation)]
    timing = time_sampler_workload(torch, package, sampler, batches, params, steps, 0.15)
    needs_exact = bool(np.any((params["temperature"] > 0) & ((params["top_k"] == 0) | (params["top_k"] > package.TOPK_FAST_MAX))))
    entry = {"workload": description + (f"; timed on {timed_rows} rows ({rows} distinct rows tiled)" if timed_rows != rows else ""), "dtype": dtype_label,
             "ms_per_step": timing["overlapped"]["ms_per_step"], "ms_per_step_single_launch": timing["single_launch"]["ms_per_step"],
             "rows_per_s": timed_rows / (timing["overlapped"]["ms_per_step"] * 1e-3),
             "frac": bytes_per_step / (timing["overlapped"]["ms_per_step"] * 1e-3) / 1e9 / peak,
             "frac_single_launch": bytes_per_step / (timing["single_launch"]["ms_per_step"] * 1e-3) / 1e9 / peak,
             "kernels_per_step": 2 if needs_exact else 1,
             "token_ids_equal": f"{agree}/{rows}", "oracle": oracle.kind}
    sampler.close()
    del batches, device
    torch.cuda.empty_cache()
    return entry


# ---- sharded workloads (N > 1) ---------------------------------------------------------


def sharded_config4(torch, dist, package, workloads, parallel, world, rank, local_rank, steps, peak):
    """Config 4, strong scaling: 8192 rows split into contiguous blocks of 8192 / world rows, no collective."""
    total_rows, vocab = 8192, 201088
    begin, end = parallel.shard_range(total_rows, world, rank)
    mine = end - begin
    (logits, params), _, description = generate(package, workloads, "config4", rows=CONFIG4_DISTINCT_ROWS)
    device = to_device(torch, logits)
    repeat = (mine + CONFIG4_DISTINCT_ROWS - 1) // CONFIG4_DISTINCT_ROWS
    device = device.repeat(repeat, 1)[:mine].contiguous()
    shard_params = np.tile(params, repeat)[:mine]
    shard_params["row_id"] = np.arange(begin, end, dtype=np.uint64)
    sampler = package.Sampler(max_rows=mine, max_vocab=vocab, device=local_rank)
    batches = [device, device.roll(1, 0).contiguous()]
    out = sampler.sample_batch(batches[0], shard_params)
    torch.cuda.synchronize()

    def step(i):
        sampler.sample_batch(batches[i % 2], None, step_offset=i, out=out)

    for i in range(3):
        step(i)
    ms, timed, _, graph = time_step_graph(torch, step, steps, 8, 0.2, barrier=dist.barrier)
    del graph
    elapsed = torch.tensor([ms], dtype=torch.float64, device="cuda")
    gathered = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
    dist.all_gather(gathered, elapsed)
    per_rank = [float(t.item()) for t in gathered]
    worst = max(per_rank)
    sampler.close()
    del batches, device
    torch.cuda.empty_cache()
    bytes_total = total_rows * vocab * 2
    return {"workload": description + f"; {CONFIG4_DISTINCT_ROWS} distinct rows tiled", "sharding": f"rows over {world} GPUs, {mine} rows per rank, no collective",
            "scaling": "strong", "ms_per_step": worst, "rows_per_s": total_rows / (worst * 1e-3), "per_rank_ms_per_step": per_rank,
            "frac_of_aggregate_peak": bytes_total / (worst * 1e-3) / 1e9 / (peak * world), "timed_steps": timed}


def sharded_config5a(torch, dist, package, workloads, parallel, world, rank, local_rank, steps, peak):
    """Config 5a across the ranks: each owns a vocabulary slice, finds its Top-K candidates, the k records
    per row are all-gathered (NCCL) and merged.  The three operations of a step are captured in one CUDA graph."""
    (logits, params), _, description = generate(package, workloads, "config5a")
    rows, vocab = logits.shape
    top_k = 64
    begin, end = parallel.vocab_shard_range(vocab, world, rank)
    slices = [torch.from_numpy(np.ascontiguousarray(np.roll(logits, shift, axis=0)[:, begin:end])).cuda() for shift in range(2)]
    sampler = package.Sampler(max_rows=rows, max_vocab=end - begin, device=local_rank)
    local = torch.empty((rows, top_k), dtype=torch.int64, device="cuda")
    gathered = torch.empty((world * rows, top_k), dtype=torch.int64, device="cuda")
    out = None

    def step(i, first=False):
        nonlocal out
        sampler.local_candidates(slices[i % 2], begin, top_k, out=local)
        dist.all_gather_into_tensor(gathered, local)
        out = sampler.merge_candidates(gathered.view(world, rows, top_k), params if first else None, top_k, step_offset=i, out=out)

    step(0, first=True)
    torch.cuda.synchronize()
    for i in range(1, 4):
        step(i)
    torch.cuda.synchronize()
    # parity of all rows of batch 0 at step offset 0
    step(0)
    torch.cuda.synchronize()
    tokens = out["token"].cpu().numpy().copy()
    # the three pieces on their own, direct calls
    pieces = {}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for label, call in (("local_candidates_ms", lambda i: sampler.local_candidates(slices[i % 2], begin, top_k, out=local)),
                        ("all_gather_ms", lambda i: dist.all_gather_into_tensor(gathered, local)),
                        ("merge_ms", lambda i: sampler.merge_candidates(gathered.view(world, rows, top_k), None, top_k, step_offset=i, out=out))):
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                call(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for i in range(16):
                call(i)
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        start.record()
        for _ in range(8):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        pieces[label] = start.elapsed_time(stop) / (8 * 16)
        del graph
    ms, timed, _, graph = time_step_graph(torch, step, steps, 16, 0.2, barrier=dist.barrier)
    del graph
    elapsed = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    worst = float(elapsed.item())
    for label in list(pieces):
        value = torch.tensor([pieces[label]], dtype=torch.float64, device="cuda")
        dist.all_reduce(value, op=dist.ReduceOp.MAX)
        pieces[label] = float(value.item())
    entry = None
    if rank == 0:
        from oracle import oracle as oracle_module
        oracle = oracle_module.best()
        want = oracle_tokens(oracle, package, logits, params, 0, rows, host_thread_count())
        agree = int(np.sum(tokens == want["token"]))
        bytes_per_step = rows * vocab * 4
        entry = {"workload": description.replace(" (single GPU)", ""), "sharding": f"vocab over {world} GPUs, all-gather of {rows}x{top_k} 8-byte records per rank",
                 "launch": "one CUDA graph per 16 steps: local candidates kernel, NCCL all-gather, merge kernel", "scaling": "strong",
                 "ms_per_step": worst, "rows_per_s": rows / (worst * 1e-3), "pieces_alone": pieces,
                 "frac_of_aggregate_peak": bytes_per_step / (worst * 1e-3) / 1e9 / (peak * world),
                 "token_ids_equal": f"{agree}/{rows}", "oracle": oracle.kind, "timed_steps": timed}
    sampler.close()
    return entry


def run_vocab_sharded_bench(args):
    """`--workload config5a --sharding vocab`: only the vocabulary-sharded workload, one JSON line."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), rank=rank, world_size=world, timeout=GROUP_TIMEOUT)
    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    parallel = __import__(graft.PACKAGE_NAME + ".parallel", fromlist=["parallel"])
    peak, _ = measured_peak()
    entry = sharded_config5a(torch, dist, package, workloads, parallel, world, rank, local_rank, min(args.steps, 512), peak)
    if rank == 0:
        line = {"metric": "vocab-sharded sampled rows/s at vocab 1048576, batch 64", "value": entry["rows_per_s"], "unit": "rows/s", "n_gpus": world,
                "steps": entry["timed_steps"], "warmup": args.warmup, "ms_per_step": entry["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "dtype": "f32", "data": "synthetic", "config": entry, "gpu_launches": 2 * entry["timed_steps"]}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--workload", default="headline", choices=sorted(WORKLOADS) + ["config5b", "speculative"])
    parser.add_argument("--sharding", default="rows", choices=["rows", "vocab"], help="vocab: config 5a split by vocabulary slice with a candidate all-gather")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--e2e-steps", type=int, default=20)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-workloads", action="store_true", help="skip the table of the other benchmark configurations")
    parser.add_argument("--no-graph", action="store_true", help="issue every step as a direct call instead of replaying a CUDA graph (for ncu captures)")
    parser.add_argument("--no-overlap", action="store_true", help="launch every step strictly after the previous one (no programmatic dependent launch)")
    parser.add_argument("--rows", type=int, default=None, help="override the workload's row count (small ncu captures)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "config5b":
        return run_router_bench(args)
    if args.workload == "speculative":
        return run_speculative_bench(args)
    if args.sharding == "vocab":
        return run_vocab_sharded_bench(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_numa_node(local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a collective left unmatched ends the run after four minutes instead of the default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=GROUP_TIMEOUT)
    barrier = dist.barrier if distributed else None

    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    parallel = __import__(graft.PACKAGE_NAME + ".parallel", fromlist=["parallel"])
    (logits, params), dtype_label, description = generate(package, workloads, args.workload, rank, rows=args.rows)
    rows, vocab = logits.shape
    element = logits.itemsize
    bytes_per_step = rows * vocab * element  # one logits read per row
    peak, peak_source = measured_peak()

    sampler = package.Sampler(max_rows=rows, max_vocab=vocab, device=local_rank)

    # distinct resident batches, rotated so that consecutive steps never read the same bytes
    # (each batch is also larger than the 126 MB L2 for the headline shape)
    rotation = 4 if bytes_per_step * 4 <= 16 << 30 else 2
    generator_state = np.random.default_rng([rank, 991])
    permutations = [np.arange(rows)] + [generator_state.permutation(rows) for _ in range(rotation - 1)]
    base = to_device(torch, logits)
    batches = [base] + [base[torch.from_numpy(p).cuda()].contiguous() for p in permutations[1:]]
    first = sampler.sample_batch(batches[0], params)  # uploads the per-row parameters once; later calls reuse them
    torch.cuda.synchronize()
    needs_exact = bool(np.any((params["temperature"] > 0) & ((params["top_k"] == 0) | (params["top_k"] > package.TOPK_FAST_MAX))))
    launches_per_step = 2 if needs_exact else 1

    # every step of a graph writes its own output buffers, so that tokens produced inside the
    # timed region can be checked afterwards
    chunk = min(args.steps, 64) if not args.no_graph else 1
    outs = [fresh_outputs(torch, rows) for _ in range(max(chunk, 1))]

    def step(i):
        sampler.sample_batch(batches[i % rotation], None, step_offset=i, out=outs[i % len(outs)])

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    clocks = ClockSampler(local_rank)
    run = {"numa": numa, "l2": f"{rotation} distinct resident batches of {bytes_per_step / 1e6:.0f} MB rotated, each step reads a different one"}
    if args.no_graph:
        # direct calls, no minimum duration: the form the ncu captures use
        sampler.set_overlap(not args.no_overlap)
        start_event, stop_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if barrier:
            barrier()
        torch.cuda.synchronize()
        clocks.start()
        start_event.record()
        for i in range(args.steps):
            step(i)
        stop_event.record()
        torch.cuda.synchronize()
        clocks.stop()
        ms_main, timed_steps, replays = start_event.elapsed_time(stop_event) / args.steps, args.steps, 0
        ms_single = ms_main
        run["launch"] = "direct calls"
    else:
        # Steps are independent batches, so their launches may overlap (programmatic dependent
        # launch): the serial tail of step i (select, sort, draw) runs while step i+1 streams.
        sampler.set_overlap(not args.no_overlap)
        ms_main, timed_steps, replays, main_graph = time_step_graph(torch, step, args.steps, chunk, MIN_TIMED_SECONDS, clocks=clocks, barrier=barrier)
        torch.cuda.synchronize()
        inside = [{k: v.clone() for k, v in outs[j].items() if v is not None} for j in (chunk - 2, chunk - 1)] if chunk >= 2 else []
        inside_steps = [chunk - 2, chunk - 1] if chunk >= 2 else []
        del main_graph
        # the same steps, every launch strictly after the previous one: what one Session's decode loop sees
        sampler.set_overlap(False)
        ms_single, single_steps, _, single_graph = time_step_graph(torch, step, min(args.steps, 1024), chunk, 0.25, barrier=barrier)
        del single_graph
        run["launch"] = (f"CUDA graph of {chunk} steps replayed {replays}x" +
                         ("" if args.no_overlap else "; consecutive launches overlap (programmatic dependent launch, the batches are independent)"))
        run["single_launch"] = {"ms_per_step": ms_single, "timed_steps": single_steps, "rows_per_s": rows / (ms_single * 1e-3),
                                "note": "same graph without overlap between launches"}
    sampler.set_overlap(False)
    # one direct C-ABI call per step, host launch overhead included
    serial_steps = min(args.steps, 256)
    serial_start, serial_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    serial_start.record()
    for i in range(serial_steps):
        step(i)
    serial_stop.record()
    torch.cuda.synchronize()
    run["serialized_direct_calls"] = {"ms_per_step": serial_start.elapsed_time(serial_stop) / serial_steps,
                                      "note": "one direct C-ABI call per step, no overlap, host launch overhead included"}

    elapsed_tensor = torch.tensor([ms_main], dtype=torch.float64, device="cuda")
    per_rank_ms = [ms_main]
    if distributed:
        gathered = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
        dist.all_gather(gathered, elapsed_tensor)
        per_rank_ms = [float(t.item()) for t in gathered]
    ms_per_step = max(per_rank_ms)
    total_rows = rows * world
    value = total_rows / (ms_per_step * 1e-3)

    # ---- end to end through the host-buffer entry point --------------------------
    pinned = []
    for b in range(2):
        tensor = torch.empty(logits.shape, dtype=torch.int16 if logits.dtype == np.uint16 else torch.float32).pin_memory()
        source = logits if b == 0 else np.roll(logits, 1, axis=0)
        tensor.numpy()[...] = source.view(np.int16) if logits.dtype == np.uint16 else source
        pinned.append(tensor)
    host_out = {"token": np.empty(rows, np.int32), "probability": np.empty(rows, np.float32), "flags": np.empty(rows, np.uint32),
                "status": np.empty(rows, np.int32)}
    dtype_code = package.DTYPE_F32 if logits.dtype == np.float32 else package.DTYPE_BF16
    e2e_steps = max(3, min(args.e2e_steps, args.steps))
    for b in range(2):
        sampler.sample_host_raw(pinned[b].data_ptr(), dtype_code, rows, vocab, params, host_out)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e2e_start = time.perf_counter()
    for i in range(e2e_steps):
        sampler.sample_host_raw(pinned[i % 2].data_ptr(), dtype_code, rows, vocab, params, host_out)  # synchronous
    e2e_elapsed = time.perf_counter() - e2e_start
    e2e_tensor = torch.tensor([e2e_elapsed], dtype=torch.float64, device="cuda")
    if distributed:
        dist.all_reduce(e2e_tensor, op=dist.ReduceOp.MAX)
    e2e_value = total_rows * e2e_steps / float(e2e_tensor.item())
    h2d_bytes = bytes_per_step + params.nbytes
    d2h_bytes = rows * (4 + 4 + 4 + 4)
    del pinned

    # ---- end to end with the logits left on the device: only the sampled rows come back ----
    results_pinned = torch.empty(rows * package.SAMPLED_ROW_DTYPE.itemsize, dtype=torch.uint8).pin_memory()
    results = results_pinned.numpy().view(package.SAMPLED_ROW_DTYPE)
    sampler.sample_tokens(batches[0], params, results=results)
    device_steps = max(e2e_steps, 200)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    device_start = time.perf_counter()
    for i in range(device_steps):
        sampler.sample_tokens(batches[i % rotation], None, step_offset=i, results=results)  # synchronous
    device_elapsed = time.perf_counter() - device_start
    device_tensor = torch.tensor([device_elapsed], dtype=torch.float64, device="cuda")
    if distributed:
        dist.all_reduce(device_tensor, op=dist.ReduceOp.MAX)
    e2e_device_value = total_rows * device_steps / float(device_tensor.item())

    # ---- sharded workloads: every rank takes part -----------------------------------
    sharded = {}
    if distributed and args.workload == "headline" and not args.no_workloads:
        sharded["config4"] = sharded_config4(torch, dist, package, workloads, parallel, world, rank, local_rank, 64, peak)
        entry = sharded_config5a(torch, dist, package, workloads, parallel, world, rank, local_rank, 256, peak)
        if entry is not None:
            sharded["config5a"] = entry

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return 0

    achieved = bytes_per_step / (ms_main * 1e-3) / 1e9  # this rank's kernel stream
    achieved_single = bytes_per_step / (ms_single * 1e-3) / 1e9
    traffic, traffic_source = captured_traffic(args.workload)
    config = workload_config(args.workload, world)
    if args.rows is not None:
        config["rows_per_gpu"] = rows
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_label,
        "data": "synthetic", "config": config, "run": run,
        "timed_steps": timed_steps, "repeats": replays,
        "clocks": clocks.summary("timed region"),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": int(d2h_bytes), "steps": e2e_steps,
                "path": "moe_sample_batch_host, pinned host logits; PCIe-bound (about 54 GB/s per GPU on this box, shared by the GPUs of a host)"},
        "e2e_device_logits": {"value": e2e_device_value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": int(rows * 16), "steps": device_steps,
                              "path": "moe_sample_tokens: logits stay on the device, one 16-byte record per row returns to page-locked host memory; synchronous call per step"},
        "gpu_launches": launches_per_step * timed_steps,
        "per_rank_ms_per_step": per_rank_ms,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "achieved_single_launch": achieved_single, "frac_single_launch": achieved_single / peak,
                     "traffic": traffic, "traffic_source": traffic_source,
                     "kernel": "sample_rows_kernel", "algorithmic_bytes_per_launch": bytes_per_step, "peak_source": peak_source},
    }
    if sharded:
        line["config"]["sharded"] = sharded

    from oracle import oracle as oracle_module
    oracle = oracle_module.best()
    threads = host_thread_count()
    if not args.no_graph and inside_steps and not args.no_cpu_baseline:
        # tokens written inside the timed (overlapped) region by the last two steps of the last replay
        agree = 0
        checked = 0
        for buffers, index in zip(inside, inside_steps):
            source = logits[permutations[index % rotation]]
            want = oracle_tokens(oracle, package, source, params, index, rows, threads)
            agree += int(np.sum(buffers["token"].cpu().numpy() == want["token"]))
            checked += rows
        line["timed_region_token_ids_equal"] = f"{agree}/{checked}"
    if world == 1 and not args.no_cpu_baseline:
        uniforms = np.array([package.philox_uniform(p["seed"], p["row_id"], p["step"]) for p in params], dtype=np.float32)
        # about 10-30 s of CPU work: 25 ms per row single-threaded at this vocabulary
        probe_rows = min(rows, max(threads, 16))
        rate, probe_elapsed, _ = cpu_sampler_rate(oracle, logits, params, uniforms, probe_rows, threads)
        target_rows = int(min(rows, max(probe_rows, rate * 3.0)))  # ~3 s of wall clock on all threads
        rate, elapsed, result = cpu_sampler_rate(oracle, logits, params, uniforms, target_rows, threads)
        agree = int(np.sum(first["token"].cpu().numpy()[:target_rows] == result["token"]))
        line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": threads, "kind": oracle.kind,
                                "sample": f"first {target_rows} of {rows} rows, {threads} host threads over independent rows, {elapsed:.2f} s wall",
                                "token_ids_equal_to_gpu": f"{agree}/{target_rows}"}
    sampler.close()
    del batches, base
    torch.cuda.empty_cache()
    if world == 1 and args.workload == "headline" and not args.no_workloads and not args.no_graph:
        table = {}
        for name in ("headline_bf16", "config2", "config3", "config4", "config5a"):
            try:
                table[name] = side_workload(torch, package, workloads, oracle, name, 64, peak, threads)
            except Exception as error:  # one workload failing must not lose the line
                table[name] = {"error": f"{type(error).__name__}: {error}"}
        for name, function in (("config5b", run_router_bench), ("speculative", run_speculative_bench)):
            try:
                entry = function(argparse.Namespace(steps=128, warmup=3), as_dict=True)
                table[name] = {k: entry[k] for k in entry if k in ("metric", "value", "unit", "ms_per_step", "regroup_gather", "routes_equal_to_reference",
                                                                  "results_equal_to_reference", "cpu_baseline", "batched")}
            except Exception as error:
                table[name] = {"error": f"{type(error).__name__}: {error}"}
        line["config"]["workloads"] = table
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
