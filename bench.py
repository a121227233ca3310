#!/usr/bin/env python
"""Benchmark of the batched sampler hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the sampler over one batch of synthetic logits.  The
default workload is the headline shape: 256 rows x vocab 201088 fp32 logits
with the config-1 parameters (T=0.7, top_k=50, top_p=0.9, min_p=0.05), rows
drawn as 3*N(0,1) plus 32 boosted entries and forced duplicates.  With N > 1
(launched by torch.distributed.run) every rank samples its own 256 rows —
rows are independent, so there is no data-path collective (weak scaling).

One JSON line is printed by rank 0:
  value      rows/s with logits and parameters resident in HBM (CUDA events over
             the K timed steps, max over ranks)
  e2e        rows/s through moe_sample_batch_host: pinned host logits in, host
             results out, copies inside the timed region
  roofline   achieved HBM GB/s of the streaming kernel (one logits read per row)
             against the measured copy bandwidth of this pool's B200s
  cpu_baseline  the reference's own CPU sampler timed on this box's host cores
             on a bounded sample of the same workload (N=1 only)

`--impl reference` times only that CPU sampler (all host threads) and prints
the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
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

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the streaming
# kernel on the headline workload, from the ncu capture summarised in
# profiles/ (None until a capture exists for the workload).
NCU_TRAFFIC_BYTES = {
    "headline": 223_360_000,  # 216.78 MB read + 6.58 MB written (mean of two captured launches), profiles/sample_rows_kernel_f32_headline.md
}

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


def generate(package, workloads, name, rank=0):
    generator, kwargs, dtype_label, description = WORKLOADS[name]
    function = getattr(workloads, generator)
    kwargs = dict(kwargs)
    if generator in ("config1_row", "config4_heavy_tail"):
        kwargs["row_offset"] = rank * kwargs["rows"]
    return function(package.ROW_PARAMS_DTYPE, **kwargs), dtype_label, description


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
    (logits, params), dtype_label, description = generate(package, workloads, args.workload)
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
    sample = f"{rows_per_step} of {rows} rows per step, {args.steps} steps, {threads} host threads over independent rows"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_label,
        "data": "synthetic", "config": {"workload": description, "rows_per_step": rows_per_step},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": oracle.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0



def run_router_bench(args):
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

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    chunk = min(args.steps, 64)
    with torch.cuda.graph(graph):
        for i in range(chunk):
            step(i)
    graph.replay()
    torch.cuda.synchronize()
    replays = max(1, args.steps // chunk)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / (replays * chunk)
    # regroup gather of the routed hidden rows (hidden size 4096 fp32): HBM-bound copy
    gathered = sampler.regroup_gather(hidden, plan.route_token)
    torch.cuda.synchronize()
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
    got_tokens = plan.route_token.cpu().numpy().view(np.uint32)
    step(0)
    torch.cuda.synchronize()
    peak, peak_source = measured_peak()
    line = {"metric": "router tokens/s, stable Top-8 of 256 experts, sigmoid scoring, 4096 tokens", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": replays * chunk, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 5b: 4096 tokens x 256 experts fp32 N(0,1) + bias N(0,0.1), sigmoid, top_k 8, renormalised", "kernels_per_step": 3},
            "gpu_launches": 3 * replays * chunk,
            "regroup_gather": {"ms": gather_ms, "achieved_gbs": gather_bytes / (gather_ms * 1e-3) / 1e9, "peak_gbs": peak, "frac": gather_bytes / (gather_ms * 1e-3) / 1e9 / peak,
                               "shape": "32768 routes x 4096 fp32 columns"},
            "cpu_baseline": {"value": tokens / cpu_s, "unit": "tokens/s", "cores": 1, "kind": oracle.kind, "sample": "the whole 4096-token call, single thread (the reference dispatcher is single-threaded)"},
            "routes_equal_to_reference": bool(np.array_equal(plan.route_token.cpu().numpy().view(np.uint32), want["token"]) and got_tokens.size == want["token"].size)}
    print(json.dumps(line), flush=True)
    sampler.close()
    return 0


def run_speculative_bench(args):
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
    steps = min(args.steps, 512)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        sampler.speculative_verify(*device_cases[i % 4], params, out=out, sync=False)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    line = {"metric": "speculative verifications/s, 4 proposed tokens, vocab 201088", "value": 1e3 / ms, "unit": "verifications/s", "n_gpus": 1,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "5 target + 4 draft rows x 201088 fp32 2.5*N(0,1) (draft = target + noise), T=1 top_k=40 top_p=0.95; direct C-ABI calls, "
                                   "device-resident logits, 4 cases rotated", "kernels_per_step": 3, "bytes_read_per_step": 9 * vocab * 4},
            "gpu_launches": 3 * steps,
            "cpu_baseline": {"value": len(cases) / t_cpu, "unit": "verifications/s", "cores": 1, "kind": oracle.kind,
                             "sample": f"{len(cases)} verifications, single thread (a Session verifies on its own thread)"},
            "results_equal_to_reference": f"{equal}/{len(cases)}"}
    print(json.dumps(line), flush=True)
    sampler.close()
    return 0


def run_vocab_sharded_bench(args):
    """Config 5a across N GPUs: each rank owns a vocabulary slice, all-gathers k candidates per row, merges."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    parallel = __import__(graft.PACKAGE_NAME + ".parallel", fromlist=["parallel"])
    logits, params = workloads.config5a_large_vocab(package.ROW_PARAMS_DTYPE)      # every rank builds the same matrix and keeps its slice
    rows, vocab = logits.shape
    top_k = 64
    begin, end = parallel.vocab_shard_range(vocab, world, rank)
    slices = [torch.from_numpy(np.ascontiguousarray(np.roll(logits, shift, axis=0)[:, begin:end])).cuda() for shift in range(4)]
    sampler = package.Sampler(max_rows=rows, max_vocab=end - begin, device=local_rank)

    def step(i):
        local = sampler.local_candidates(slices[i % 4], begin, top_k)
        gathered = parallel.all_gather_candidates(local) if world > 1 else local.unsqueeze(0)
        return sampler.merge_candidates(gathered, params if i == 0 else None, top_k, step_offset=i)

    out = step(0)
    for i in range(1, args.warmup):
        out = step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(args.steps):
        step(args.warmup + i)
    stop.record()
    torch.cuda.synchronize()
    elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms = float(elapsed.item()) / args.steps
    check = step(0)
    torch.cuda.synchronize()
    if rank == 0:
        from oracle import oracle as oracle_module
        oracle = oracle_module.best()
        sample_rows = 8
        uniforms = np.array([package.philox_uniform(p["seed"], p["row_id"], p["step"]) for p in params[:sample_rows]], dtype=np.float32)
        want = oracle.sample_batch(logits[:sample_rows], params["temperature"][:sample_rows], params["top_k"][:sample_rows], params["top_p"][:sample_rows],
                                   params["min_p"][:sample_rows], uniforms)
        agree = int(np.sum(check["token"].cpu().numpy()[:sample_rows] == want["token"]))
        peak, _ = measured_peak()
        bytes_per_step = rows * vocab * 4
        line = {"metric": "vocab-sharded sampled rows/s at vocab 1048576, batch 64", "value": rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "f32", "data": "synthetic",
                "config": {"workload": "config 5a: 64 rows x vocab 1048576 fp32, top_k 64 top_p 0.9", "sharding": f"vocab over {world} GPUs, all-gather of {rows}x{top_k} 8-byte records",
                           "launch": "direct calls (local candidates kernel, NCCL all-gather, merge kernel)"},
                "roofline": {"bound": "hbm", "achieved": bytes_per_step / (ms * 1e-3) / 1e9, "peak": peak * world, "unit": "GB/s",
                             "frac": bytes_per_step / (ms * 1e-3) / 1e9 / (peak * world)},
                "gpu_launches": (2 + (1 if world > 1 else 0)) * args.steps, "token_ids_equal_to_reference": f"{agree}/{sample_rows}"}
        print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
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
    parser.add_argument("--no-graph", action="store_true", help="issue every step as a direct call instead of replaying a CUDA graph")
    parser.add_argument("--no-overlap", action="store_true", help="launch every step strictly after the previous one (no programmatic dependent launch)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.workload == "config5b":
        return run_router_bench(args)
    if args.workload == "speculative":
        return run_speculative_bench(args)
    if args.sharding == "vocab":
        return run_vocab_sharded_bench(args)
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    package = graft.load_package()
    workloads = __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])
    (logits, params), dtype_label, description = generate(package, workloads, args.workload, rank)
    rows, vocab = logits.shape
    element = 4 if logits.dtype == np.float32 else 2
    bytes_per_step = rows * vocab * element  # one logits read per row

    sampler = package.Sampler(max_rows=rows, max_vocab=vocab, device=local_rank)

    def to_device(array):
        if array.dtype == np.uint16:
            return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
        return torch.from_numpy(array).cuda()

    # distinct resident batches, rotated so that consecutive steps never read the same bytes
    # (each batch is also larger than the 126 MB L2 for the headline shape)
    rotation = 4 if bytes_per_step * 4 <= 16 << 30 else 2
    batches = [to_device(logits)]
    generator_state = np.random.default_rng([rank, 991])
    for _ in range(rotation - 1):
        permutation = torch.from_numpy(generator_state.permutation(rows)).cuda()
        batches.append(batches[0][permutation].contiguous())
    out = sampler.sample_batch(batches[0], params)  # uploads the per-row parameters once; later calls reuse them
    torch.cuda.synchronize()
    needs_exact = bool(np.any((params["temperature"] > 0) & ((params["top_k"] == 0) | (params["top_k"] > package.TOPK_FAST_MAX))))
    launches_per_step = 2 if needs_exact else 1

    def step(i):
        sampler.sample_batch(batches[i % rotation], None, step_offset=i, out=out)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    # Steps are independent batches, so their launches may overlap (programmatic dependent
    # launch): the serial tail of step i (select, sort, draw) runs while step i+1 streams.
    sampler.set_overlap(not args.no_overlap)
    # The kernels of a step take tens of microseconds, less than one Python ->
    # ctypes call, so the timed loop replays a CUDA graph of `chunk` consecutive
    # steps (captured from the same C-ABI calls) and issues the remainder directly.
    chunk = min(args.steps, 64 if not args.no_graph else 0)
    graph = None
    if chunk > 1:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(chunk):
                step(args.warmup + i)
        graph.replay()
        torch.cuda.synchronize()
    replays = args.steps // chunk if graph is not None else 0
    remainder = args.steps - replays * chunk if graph is not None else args.steps
    # the steps that do not fill a whole chunk get a graph of their own, so that the timed
    # region holds no per-step host work at all
    tail_graph = None
    if graph is not None and remainder > 1:
        tail_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(tail_graph):
            for i in range(remainder):
                step(args.warmup + i)
        tail_graph.replay()
        torch.cuda.synchronize()

    clocks = ClockSampler(local_rank)
    start_event = torch.cuda.Event(enable_timing=True)
    stop_event = torch.cuda.Event(enable_timing=True)
    if distributed:
        dist.barrier()
    torch.cuda.synchronize()
    clocks.start()
    start_event.record()
    for _ in range(replays):
        graph.replay()
    if tail_graph is not None:
        tail_graph.replay()
    else:
        for i in range(remainder):
            step(args.warmup + i)
    stop_event.record()
    torch.cuda.synchronize()
    clocks.stop()
    if distributed:
        dist.barrier()
    elapsed_ms = start_event.elapsed_time(stop_event)
    # the same steps strictly one after the other, for the record (latency of a single step)
    sampler.set_overlap(False)
    serial_steps = min(args.steps, 256)
    serial_start = torch.cuda.Event(enable_timing=True)
    serial_stop = torch.cuda.Event(enable_timing=True)
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    serial_start.record()
    for i in range(serial_steps):
        step(args.warmup + i)
    serial_stop.record()
    torch.cuda.synchronize()
    serial_ms_per_step = serial_start.elapsed_time(serial_stop) / serial_steps
    clock_where = "timed region"
    if len(clocks.samples) < 5:
        # the timed region was shorter than a few NVML polls: sample the same loop again, untimed
        clocks.start()
        deadline = time.perf_counter() + 0.4
        i = 0
        while time.perf_counter() < deadline:
            for _ in range(50):
                step(i)
                i += 1
            torch.cuda.synchronize()
        clocks.stop()
        clock_where = "same loop repeated right after the timed region (region shorter than the polling period)"
    elapsed_tensor = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
    if distributed:
        dist.all_reduce(elapsed_tensor, op=dist.ReduceOp.MAX)
    worst_ms = float(elapsed_tensor.item())
    per_rank_ms = [elapsed_ms / args.steps]
    if distributed:
        gathered = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
        dist.all_gather(gathered, torch.tensor([elapsed_ms / args.steps], dtype=torch.float64, device="cuda"))
        per_rank_ms = [float(t.item()) for t in gathered]
    total_rows = rows * world
    value = total_rows * args.steps / (worst_ms * 1e-3)
    ms_per_step = worst_ms / args.steps

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
    if distributed:
        dist.barrier()
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

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return 0

    peak, peak_source = measured_peak()
    achieved = bytes_per_step / (elapsed_ms / args.steps * 1e-3) / 1e9  # this rank's kernel stream
    traffic = NCU_TRAFFIC_BYTES.get(args.workload)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_label,
        "data": "synthetic",
        "config": {"workload": description, "rows_per_gpu": rows, "vocab": vocab, "sharding": "rows" if world > 1 else "none",
                   "launch": (f"CUDA graph of {chunk} steps replayed {replays}x + " + (f"one graph of {remainder} steps" if tail_graph is not None else f"{remainder} direct calls")
                              if graph is not None else "direct calls")
                             + ("" if args.no_overlap else "; consecutive launches overlap (programmatic dependent launch, the batches are independent)"),
                   "serialized_direct_calls": {"ms_per_step": serial_ms_per_step, "rows_per_s": rows / (serial_ms_per_step * 1e-3),
                                               "note": "same steps without overlap, one direct C-ABI call per step, host launch overhead included"},
                   "l2": f"{rotation} distinct resident batches of {bytes_per_step / 1e6:.0f} MB rotated, each step reads a different one"},
        "clocks": clocks.summary(clock_where),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": int(d2h_bytes), "steps": e2e_steps,
                "path": "moe_sample_batch_host, pinned host logits"},
        "gpu_launches": launches_per_step * args.steps,
        "per_rank_ms_per_step": per_rank_ms,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                     "kernel": "sample_rows_kernel", "algorithmic_bytes_per_launch": bytes_per_step, "peak_source": peak_source},
    }

    if world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as oracle_module
        oracle = oracle_module.best()
        threads = host_thread_count()
        uniforms = np.array([package.philox_uniform(p["seed"], p["row_id"], p["step"]) for p in params], dtype=np.float32)
        # about 10-30 s of CPU work: 25 ms per row single-threaded at this vocabulary
        probe_rows = min(rows, max(threads, 16))
        rate, probe_elapsed, _ = cpu_sampler_rate(oracle, logits, params, uniforms, probe_rows, threads)
        target_rows = int(min(rows, max(probe_rows, rate * 3.0)))  # ~3 s of wall clock on all threads
        rate, elapsed, result = cpu_sampler_rate(oracle, logits, params, uniforms, target_rows, threads)
        tokens = out["token"].cpu().numpy()
        # the last resident batch order differs from `logits`; check parity on a fresh call instead
        check = sampler.sample_batch(batches[0], params)
        torch.cuda.synchronize()
        agree = int(np.sum(check["token"].cpu().numpy()[:target_rows] == result["token"]))
        line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": threads, "kind": oracle.kind,
                                "sample": f"first {target_rows} of {rows} rows, {threads} host threads over independent rows, {elapsed:.2f} s wall",
                                "token_ids_equal_to_gpu": f"{agree}/{target_rows}"}
        del tokens
    print(json.dumps(line), flush=True)
    sampler.close()
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
