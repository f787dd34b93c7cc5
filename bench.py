#!/usr/bin/env python
"""Throughput of the fused token-sampling path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one fg_cuda_sample_batch call over one batch of synthetic logits:
batch 1024 x vocabulary 151,936 fp32, Gumbel(0,1)+N(0,2^2) logits, frequency
0.5 / repetition 1.05 penalties over a 4,096-token Zipf history per row,
temperature 1.0, top-k 50, top-p 0.95 — every GPU samples its own 1024 rows
(rows are independent, so ranks share nothing: weak scaling, no collective).

The JSON line printed by rank 0 carries
  value       rows/s of the whole job, inputs resident in HBM, CUDA-event time
  e2e         the same metric through the host-buffer C-ABI entry
              (fg_cuda_sample_batch_host): pinned host inputs copied to the
              device and results copied back inside the timed region
  roofline    algorithmic bytes per launch / mean launch time, against the
              measured HBM copy bandwidth
  cpu_baseline  the CPU oracle timed on this box's host cores (N = 1 only)

--impl reference times the CPU implementation alone (the reference's own
sampler objects when oracle/_ref was built, else this repository's port of
them), with all host threads, on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS = 1024
VOCAB = 151_936
HISTORY = 4096
METRIC = "sampled_rows_per_sec"
FALLBACK_HBM_GBS = 6650.0
WORKLOAD = ("config3: batch 1024 x vocab 151936 fp32 per GPU, Gumbel(0,1)+N(0,2^2), frequency 0.5 + "
            "repetition 1.05 over 4096-token Zipf(1.0) history, T=1.0 top_k=50 top_p=0.95")


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


KERNELS = {
    # kernel name -> the committed ncu summary that holds its DRAM bytes per row
    "persistent_select_kernel<float>": "persistent_select_config3_ncu.txt",
    "stream_select_kernel<float>": "stream_select_config3_ncu.txt",
}


def kernel_taken(path: str, rows: int, sm_count: int) -> str:
    """The kernel the library launches for this workload (16-byte aligned fp32 rows, penalties
    that only lower logits): the persistent ring kernel unless the other one is asked for."""
    return "stream_select_kernel<float>" if path == "registers" else "persistent_select_kernel<float>"


def recorded_traffic_per_row(kernel: str):
    """DRAM bytes per row of the kernel, from its committed ncu summary."""
    path = ROOT / "profiles" / KERNELS[kernel]
    try:
        found = re.search(r"dram_bytes_per_row\s*=\s*([0-9.]+)", path.read_text())
        return float(found.group(1)) if found else None
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.process.terminate()  # the exact child we started
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        if self.thread:
            self.thread.join(timeout=2)
        clocks, reasons, top = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                top = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        median = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": median, "sm_max_mhz": top, "reasons": sorted(reasons),
                "samples": len(clocks)}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_arm(workload, kind: str, threads: int, repeats: int):
    """rows/s of the CPU oracle over the whole batch; best of `repeats`."""
    import numpy as np
    import oracle
    lib = oracle.load(kind)
    logits = workload.logits.cpu().numpy()
    tokens = workload.history_tokens.cpu().numpy().view(np.uint32)
    offsets = workload.history_offsets.cpu().numpy().view(np.uint64)
    uniforms = workload.uniforms.cpu().numpy()
    times, out = [], None
    for _ in range(repeats):
        begin = time.perf_counter()
        out = oracle.sample_batch(lib, logits, workload.configs, uniforms, tokens, offsets, False, threads)
        times.append(time.perf_counter() - begin)
    return workload.rows / min(times), times, out


def run_reference(args, rank: int):
    """The CPU implementation on this box's host cores (rank 0 only)."""
    if rank != 0:
        return
    import torch
    import oracle
    from flash_gordon_b200 import synth
    kind = "reference" if oracle.available("reference") else "port"
    threads = host_threads()
    workload = synth.config3(device="cpu", rows=ROWS, vocab=VOCAB, history=HISTORY)
    # each step is a bounded sample of the batch: as many of its rows as keep the whole
    # run near 90 s on these cores (all of them when the steps are few)
    _, calibration, _ = cpu_arm(workload, kind, threads, 1)
    budget_rows = int(ROWS * 90.0 / (max(args.steps, 1) * calibration[0]))
    rows_per_step = max(threads, min(ROWS, budget_rows // threads * threads))
    sample = workload.slice_rows(0, rows_per_step)
    for _ in range(min(args.warmup, 3)):
        cpu_arm(sample, kind, threads, 1)
    begin = time.perf_counter()
    for _ in range(args.steps):
        cpu_arm(sample, kind, threads, 1)
    elapsed = time.perf_counter() - begin
    value = rows_per_step * args.steps / elapsed
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "rows_per_step": rows_per_step},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                         "sample": f"the first {rows_per_step} of the batch's {ROWS} rows per step, "
                                   f"{args.steps} steps, {threads} host threads, rows in parallel"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--e2e-steps", type=int, default=10)
    parser.add_argument("--splits", type=int, default=0, help="force CTAs per row (0 = automatic)")
    parser.add_argument("--path", default="auto", choices=["auto", "registers", "ring"],
                        help="kernel: the library's choice, the register-prefetch kernel, or the "
                             "persistent ring kernel")
    parser.add_argument("--rows", type=int, default=ROWS)
    parser.add_argument("--skip-cpu", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from flash_gordon_b200 import Context, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    rows = args.rows
    # two independent input sets, alternated, each far larger than the 126 MB L2
    sets = [synth.config3(device=device, rows=rows, vocab=VOCAB, history=HISTORY, seed=303 + 1000 * rank + i)
            for i in range(2)]
    context = Context(local_rank)
    if args.splits:
        context.set_splits(args.splits)
    context.set_path({"auto": 0, "registers": 1, "ring": 2}[args.path])
    outs = [(torch.empty(rows, dtype=torch.int32, device=device),
             torch.empty(rows, dtype=torch.float32, device=device),
             torch.empty(rows, dtype=torch.int32, device=device)) for _ in sets]
    steps = [context.prepared_sample(w.logits, w.configs, w.uniforms, w.history_tokens,
                                     w.history_offsets, w.history_max, out)
             for w, out in zip(sets, outs)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        steps[i % 2]()
    barrier()
    if int(outs[0][2].max()) != 0:
        raise SystemExit("warm-up rows failed: " + str(outs[0][2].unique().tolist()))

    # ---- device-resident throughput: per-launch CUDA events on the launching stream ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches_before = context.launches
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        events[i][0].record()
        steps[i % 2]()
        events[i][1].record()
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    launch_ms = sorted(a.elapsed_time(b) for a, b in events)
    gpu_launches = context.launches - launches_before
    clocks = sampler.stop()
    if int(outs[0][2].max()) != 0 or int(outs[1][2].max()) != 0:
        raise SystemExit("timed rows failed")

    # ---- end to end: host buffers in, tokens out, through the C-ABI host entry ----
    host = sets[0].to("cpu")
    pinned = [t.pin_memory() for t in (host.logits, host.uniforms, host.history_tokens, host.history_offsets)]
    host_out = (torch.empty(rows, dtype=torch.int32).pin_memory(),
                torch.empty(rows, dtype=torch.float32).pin_memory(),
                torch.empty(rows, dtype=torch.int32).pin_memory())
    h2d = sum(t.numel() * t.element_size() for t in pinned)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step():
        result = context.sample_batch_host(pinned[0], host.configs, pinned[1], pinned[2], pinned[3],
                                           host.history_max, out=host_out)
        if result.status != 0:
            raise SystemExit(f"end-to-end step failed: {result.message}")

    for _ in range(2):
        e2e_step()
    barrier()
    e2e_begin = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()  # returns with the tokens on the host
    torch.cuda.synchronize()
    e2e_ms = 1e3 * (time.perf_counter() - e2e_begin)
    same = bool((host_out[0] == outs[0][0].cpu()).all())

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        bytes_per_row = sets[0].algorithmic_bytes_per_row()
        mean_launch_ms = sum(launch_ms) / len(launch_ms)
        achieved = rows * bytes_per_row / (mean_launch_ms * 1e-3) / 1e9
        kernel = kernel_taken(args.path, rows, torch.cuda.get_device_properties(device).multi_processor_count)
        traffic_row = recorded_traffic_per_row(kernel)
        line = {
            "metric": METRIC,
            "value": world * rows * args.steps / (elapsed_ms * 1e-3),
            "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": rows, "vocab": VOCAB, "history": HISTORY,
                       "l2": "two alternating 639 MB input sets per GPU, each larger than L2",
                       "parallelism": f"rows x{world} (no collective)"},
            "e2e": {"value": world * rows * args.e2e_steps / (e2e_ms * 1e-3), "unit": "rows/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
                    "matches_device_path": same},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": kernel,
                         "algorithmic_bytes_per_row": bytes_per_row,
                         "launch_ms": {"mean": mean_launch_ms, "median": launch_ms[len(launch_ms) // 2],
                                       "min": launch_ms[0]},
                         "traffic": None if traffic_row is None else traffic_row * rows},
        }
        if world == 1 and not args.skip_cpu:
            import oracle
            kind = "reference" if oracle.available("reference") else "port"
            threads = host_threads()
            value, samples, expected = cpu_arm(host, kind, threads, 3)
            import numpy as np
            got = outs[0][0].cpu().numpy().view(np.uint32)
            line["cpu_baseline"] = {
                "value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                "sample": f"the whole {rows}-row batch, best of 3 passes of {min(samples):.2f}-"
                          f"{max(samples):.2f} s, {threads} host threads, rows in parallel",
                "tokens_match_gpu": bool(np.array_equal(got, expected[1])),
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
