#!/usr/bin/env python
"""Throughput of the fused token-sampling path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload config5]

One step = one pass of the sampling path over one batch of synthetic logits.
Default workload (the configuration the metric is quoted on): batch 1024 x
vocabulary 151,936 fp32, Gumbel(0,1)+N(0,2^2) logits, frequency 0.5 /
repetition 1.05 penalties over a 4,096-token Zipf history per row, temperature
1.0, top-k 50, top-p 0.95.  The batch is PARTITIONED BY ROWS over the N GPUs
(strong scaling: 1024 rows in total, contiguous blocks, no data-path
collective; ranks only meet at the timing barriers).

The JSON line printed by rank 0 carries
  value         rows/s of the whole job, inputs resident in HBM, CUDA-event time,
                max over ranks
  e2e           the same metric through the host-buffer C-ABI entry
                (fg_cuda_sample_batch_host): pinned host inputs copied to the
                device and results copied back inside the timed region
  roofline      algorithmic bytes per launch / mean launch time (per-launch CUDA
                events on the launching stream), against the measured HBM copy
                bandwidth
  cpu_baseline  the CPU oracle timed on this box's host cores (N = 1 only)
  weak          (N > 1) the same kernel with 1024 rows on EVERY GPU
  sharded       (N > 1) the vocabulary-sharded mode: batch 256 x 151,936 bf16
                split by columns over the N GPUs, shard top-64, one all-gather
                of (value, index) pairs, merge and sample; microseconds per step
  latency_us    one launch of the 1-row greedy and the 64-row configurations
  t1_call_us    one fg_sampler_select / fg_sampler_apply_penalties call through
                the host-pointer C ABI (each is a GPU round trip)

--impl reference times the CPU implementation alone (the reference's own
sampler objects when oracle/_ref was built, else this repository's port of
them), with all host threads, on the same workload; it never loads the CUDA
library.
"""
from __future__ import annotations

import argparse
import hashlib
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
SEED = 303
METRIC = "sampled_rows_per_sec"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024
WORKLOADS = {
    "config3": ("config3: batch 1024 x vocab 151936 fp32 partitioned by rows over the GPUs, "
                "Gumbel(0,1)+N(0,2^2), frequency 0.5 + repetition 1.05 over 4096-token Zipf(1.0) "
                "history, T=1.0 top_k=50 top_p=0.95"),
    "config5": ("config5: batch 4096 x vocab 151936 fp32 partitioned by rows over the GPUs, "
                "N(0,0.5^2), presence 0.5 + frequency 0.5 over 32768-token uniform history, "
                "T=1.2 top_p=0.99, no top-k cut"),
}


def workload_config(name: str, world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    rows = ROWS if name == "config3" else 4096
    return {"workload": WORKLOADS[name], "rows_total": rows, "vocab": VOCAB,
            "history": HISTORY if name == "config3" else 32768, "seed": SEED,
            "l2": "input sets rotated so that consecutive steps never read the same set; the "
                  "sets together are more than three times the 126 MB L2",
            "parallelism": f"rows partitioned x{world} (no collective on the data path)"}


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
    "nucleus_select_kernel": "nucleus_select_config5_ncu.txt",
}


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
                self.samples.append((time.perf_counter(), parts))

    def wait_first(self, seconds: float = 5.0):
        """Blocks until nvidia-smi has delivered its first sample (it takes a while to start)."""
        limit = time.perf_counter() + seconds
        while self.process is not None and not self.samples and time.perf_counter() < limit:
            time.sleep(0.01)

    def stop(self, windows=()) -> dict:
        """`windows`: (begin, end) perf_counter pairs of the timed regions; the median clock
        is taken over the samples inside them (all samples if none falls inside)."""
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.process.terminate()  # the exact child we started
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        if self.thread:
            self.thread.join(timeout=2)
        inside = [p for t, p in self.samples if any(a <= t <= b + 0.02 for a, b in windows)]
        chosen = inside if inside else [p for _, p in self.samples]
        clocks, reasons, top = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in chosen:
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
                "samples": len(clocks), "samples_in_timed_regions": len(inside)}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def make_workload(name: str, device="cpu", rows=None, seed=SEED):
    from flash_gordon_b200 import synth
    if name == "config3":
        return synth.config3(device=device, rows=ROWS if rows is None else rows, vocab=VOCAB,
                             history=HISTORY, seed=seed)
    return synth.config5(device=device, rows=4096 if rows is None else rows, vocab=VOCAB, seed=seed)


def input_record(workload) -> dict:
    """Generator, seed and SHA-256 of the input blobs (logits, history, uniforms)."""
    digest = hashlib.sha256()
    for tensor in (workload.logits, workload.history_tokens, workload.history_offsets, workload.uniforms):
        if tensor is not None:
            digest.update(tensor.cpu().contiguous().numpy().tobytes())
    return {"generator": f"flash_gordon_b200.synth.{workload.name} on the host, torch CPU generator",
            "seed": workload.meta.get("seed"), "rows": workload.rows, "sha256": digest.hexdigest()}


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
        out = oracle.sample_batch(lib, logits, workload.configs, uniforms, tokens, offsets,
                                  workload.allow_no_topk, threads)
        times.append(time.perf_counter() - begin)
    return workload.rows / min(times), times, out


def run_reference(args, rank: int):
    """The CPU implementation on this box's host cores (rank 0 only).  Imports the input
    generator and the oracle; never the CUDA library."""
    if rank != 0:
        return
    import oracle
    kind = "reference" if oracle.available("reference") else "port"
    threads = host_threads()
    rows_total = ROWS if args.workload == "config3" else 4096
    # a bounded sample: the first rows of the batch, as many as keep the whole run near 90 s
    probe_rows = min(rows_total, max(threads, 64))
    workload = make_workload(args.workload, rows=rows_total if args.workload == "config3" else probe_rows)
    probe = workload.slice_rows(0, probe_rows)
    _, calibration, _ = cpu_arm(probe, kind, threads, 1)
    per_row = calibration[0] / probe_rows
    budget_rows = int(90.0 / (max(args.steps + min(args.warmup, 3), 1) * per_row))
    rows_per_step = max(threads, min(workload.rows, budget_rows // threads * threads))
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
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.workload, args.gpus),
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                         "sample": f"the first {rows_per_step} of the batch's {rows_total} rows per step, "
                                   f"{args.steps} steps, {threads} host threads, rows in parallel"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_steps(steps, count, barrier, torch):
    """`count` launches rotating through `steps`; returns (whole-region ms, perf_counter window)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    begin = time.perf_counter()
    start.record()
    for i in range(count):
        steps[i % len(steps)]()
    stop.record()
    barrier()
    return start.elapsed_time(stop), (begin, time.perf_counter())


def launch_times(steps, count, torch):
    """Per-launch CUDA-event durations (ms) over `count` launches on the launching stream."""
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(count)]
    torch.cuda.synchronize()
    for i in range(count):
        events[i][0].record()
        steps[i % len(steps)]()
        events[i][1].record()
    torch.cuda.synchronize()
    return sorted(a.elapsed_time(b) for a, b in events)


def prepared(context, sets, torch, device):
    outs = [(torch.empty(w.rows, dtype=torch.int32, device=device),
             torch.empty(w.rows, dtype=torch.float32, device=device),
             torch.empty(w.rows, dtype=torch.int32, device=device)) for w in sets]
    steps = [context.prepared_sample(w.logits, w.configs, w.uniforms, w.history_tokens,
                                     w.history_offsets, w.history_max, out, allow_no_topk=w.allow_no_topk)
             for w, out in zip(sets, outs)]
    return steps, outs


def rotation(per_set_bytes: int) -> int:
    """How many input sets to rotate through so that they total more than 3x the L2."""
    return max(2, -(-3 * L2_BYTES // max(per_set_bytes, 1)) + 1)


def sharded_record(context, world, rank, device, steps, barrier, torch, dist):
    """Config 4: batch 256 x 151,936 bf16 split by columns, shard top-64, all-gather, merge."""
    import numpy as np
    from flash_gordon_b200 import synth
    from flash_gordon_b200.dist import Communicator, shard_span
    full = synth.config4(rows=256, vocab=VOCAB)
    first, width = shard_span(VOCAB, world, rank)
    communicator = Communicator(context)
    # rotate shards so that the logits come from HBM: 256 x width bf16 is ~10 MB at N = 8
    mine = [full.logits[:, first:first + width].contiguous().to(device)]
    for i in range(1, rotation(mine[0].numel() * 2)):
        mine.append((torch.randn(256, width, device=device) * 4.0).to(torch.bfloat16))
    uniforms = full.uniforms.to(device)
    out = (torch.empty(256, dtype=torch.int32, device=device), torch.empty(256, dtype=torch.float32, device=device),
           torch.empty(256, dtype=torch.int32, device=device))
    def agree(failed: bool, what: str):
        """Every rank leaves together when any of them failed (nobody is left in a collective)."""
        flag = torch.tensor([1 if failed else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag[0]) != 0:
            raise RuntimeError(what)

    result = communicator.sample_vocab_sharded(mine[0], full.configs, uniforms, VOCAB, 64, out=out)
    agree(result.status != 0, f"sharded step failed: {result.message}")
    record = {"workload": "config4: batch 256 x vocab 151936 bf16 split by columns over the GPUs, "
                          "N(0,4^2), shard top-64, all-gather of (fp32 value, int32 id), merge, "
                          "T=0.8 top_p=0.9 top_k=64", "columns_per_gpu": width,
              "exchange": "ncclAllGather inside fg_dist_sample_vocab_sharded (C ABI)"}
    if rank == 0:
        import oracle
        kind = "reference" if oracle.available("reference") else "port"
        lib = oracle.load(kind)
        want = oracle.sample_batch(lib, full.logits.view(torch.int16).numpy().view(np.uint16), full.configs,
                                   full.uniforms.numpy(), None, None, False, host_threads())
        record["tokens_match_unsharded_oracle"] = bool(
            np.array_equal(result.tokens.cpu().numpy().view(np.uint32), want[1]) and
            np.array_equal(result.token_logits.cpu().numpy().view(np.uint32), want[2].view(np.uint32)))
        record["oracle_kind"] = kind

    def timed(fused):
        """ms for `steps` asynchronous calls, one after the other, max over the ranks."""
        calls = [communicator.prepared_sample_vocab_sharded(shard, full.configs, uniforms, VOCAB, 64, out,
                                                            fused=fused) for shard in mine]
        refused = False
        for i in range(5):
            refused = calls[i % len(calls)]() != 0 or refused
        agree(refused, "a sharded step could not be enqueued" + (" (fused exchange)" if fused else ""))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(steps):
            calls[i % len(calls)]()
        stop.record()
        barrier()
        agree(int(out[2].max()) != 0, "sharded rows failed" + (" (fused exchange)" if fused else ""))
        span = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
        dist.all_reduce(span, op=dist.ReduceOp.MAX)
        return span

    total = timed(False)
    try:  # (every rank raises together, see agree(): the NCCL figures above stay)
        fused_total, fused_error = timed(True), None
    except RuntimeError as error:
        fused_total, fused_error = None, str(error)

    # the two compute steps on their own (per-launch events); the exchange is the rest
    scores = torch.empty(256, 64, dtype=torch.float32, device=device)
    ids = torch.empty(256, 64, dtype=torch.int32, device=device)
    shard_steps = [lambda i=i: context.shard_topk(mine[i], full.configs, first, VOCAB, 64, out=(scores, ids),
                                                  asynchronous=True) for i in range(len(mine))]
    for step in shard_steps:
        step()
    spans = launch_times(shard_steps, min(steps, 100), torch)
    shard_us = 1e3 * spans[len(spans) // 2]
    all_scores = scores.unsqueeze(0).repeat(world, 1, 1).contiguous()
    all_ids = torch.stack([ids + (shard_span(VOCAB, world, s)[0] - first) for s in range(world)]).contiguous()
    spans_list = [shard_span(VOCAB, world, s) for s in range(world)]
    merge_step = lambda: context.merge_select(all_scores, all_ids, 256, world, 64, [s[0] for s in spans_list],
                                              [s[1] for s in spans_list], full.configs, uniforms,
                                              asynchronous=True)
    merge_step()
    spans = launch_times([merge_step], min(steps, 100), torch)
    merge_us = 1e3 * spans[len(spans) // 2]
    us_per_step = 1e3 * float(total[0]) / steps
    record.update({"us_per_step": us_per_step, "steps": steps,
                   "rows_per_sec": 256 * steps / (float(total[0]) * 1e-3),
                   "shard_kernel_us": shard_us, "merge_us": merge_us,
                   "exchange_us": max(0.0, us_per_step - shard_us - merge_us),
                   "fused_us_per_step": None if fused_total is None else 1e3 * float(fused_total[0]) / steps,
                   "fused_error": fused_error,
                   "fused_exchange": "fg_dist_sample_vocab_sharded_fused: the shard kernel stores its pairs into "
                                     "every rank's window (CUDA IPC), the merge kernel waits for them",
                   "bytes_sent_per_rank": 256 * 64 * 8, "bytes_gathered_per_rank": 256 * 64 * 8 * world})
    communicator.close()
    return record


def small_latencies(context, device, torch):
    """One launch of the 1-row greedy configuration and of the 64-row configuration (us)."""
    from flash_gordon_b200 import synth
    out = {}
    for name, make in (("config1", lambda s: synth.config1(device=device, seed=101 + s)),
                       ("config2", lambda s: synth.config2(device=device, seed=202 + s))):
        probe = make(0)
        sets = [probe] + [make(s) for s in range(1, rotation(probe.logits.numel() * 4))]
        steps, outs = prepared(context, sets, torch, device)
        for i in range(2 * len(steps)):
            steps[i % len(steps)]()
        spans = launch_times(steps, 60, torch)
        out[name] = round(1e3 * spans[len(spans) // 2], 2)
    return out


def t1_latencies():
    """One fg_sampler_select and one fg_sampler_apply_penalties call through the host-pointer
    C ABI (host arrays in and out; each stages to the GPU, launches and waits)."""
    import ctypes
    import numpy as np
    from flash_gordon_b200 import SamplerConfig, api, load_library
    lib = load_library()
    cfg = SamplerConfig.make(temperature=0.7, top_p=0.8, top_k=20, presence=1.5)
    scores = np.linspace(5.0, -1.0, 64, dtype=np.float32)
    ids = np.arange(64, dtype=np.uint32)
    for _ in range(5):
        api.select(cfg, scores.tolist(), ids.tolist(), 0.37)
    begin = time.perf_counter()
    for _ in range(200):
        api.select(cfg, scores.tolist(), ids.tolist(), 0.37)
    select_us = 1e6 * (time.perf_counter() - begin) / 200
    values = np.random.default_rng(1).standard_normal(VOCAB).astype(np.float32)
    identity = np.arange(VOCAB, dtype=np.uint32)
    counts = np.zeros(VOCAB, dtype=np.uint32)
    counts[::37] = 2
    P = ctypes.c_void_p
    call = lambda: lib.fg_sampler_apply_penalties(P(values.ctypes.data), P(identity.ctypes.data),
                                                  P(counts.ctypes.data), VOCAB, ctypes.byref(cfg))
    for _ in range(3):
        call()
    begin = time.perf_counter()
    for _ in range(50):
        call()
    return {"fg_sampler_select_64": round(select_us, 1),
            "fg_sampler_apply_penalties_vocab": round(1e6 * (time.perf_counter() - begin) / 50, 1)}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="config3", choices=sorted(WORKLOADS))
    parser.add_argument("--e2e-steps", type=int, default=10)
    parser.add_argument("--path", default="auto", choices=["auto", "registers", "ring"],
                        help="kernel: the library's choice, the register-prefetch kernel, or the "
                             "persistent ring kernel")
    parser.add_argument("--skip-cpu", action="store_true")
    parser.add_argument("--skip-extras", action="store_true",
                        help="headline, roofline and e2e only (no weak / sharded / latency records)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from flash_gordon_b200 import Context
    from flash_gordon_b200.dist import row_block

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- inputs: the canonical batch on the host (hashed), this rank's block on the device ----
    rows_total = ROWS if args.workload == "config3" else 4096
    begin_row, end_row = row_block(rows_total, world, rank)
    rows = end_row - begin_row
    if args.workload == "config3":
        canonical = make_workload("config3")
        host_block = canonical.slice_rows(begin_row, end_row)
        inputs = input_record(canonical) if rank == 0 else None
    else:
        # config 5 is 2.5 GB of logits for the whole batch: each rank makes its own block
        canonical = None
        host_block = make_workload("config5", rows=rows, seed=SEED + 7919 * rank)
        inputs = input_record(host_block) if rank == 0 else None
    first_set = host_block.to(device)
    sets = [first_set]
    per_set = first_set.logits.numel() * first_set.logits.element_size()
    for i in range(1, rotation(per_set)):
        sets.append(make_workload(args.workload, device=device, rows=rows, seed=SEED + 1000 * i + rank))
    context = Context(local_rank)
    context.set_path({"auto": 0, "registers": 1, "ring": 2}[args.path])
    steps, outs = prepared(context, sets, torch, device)

    for i in range(max(args.warmup, len(steps))):
        steps[i % len(steps)]()
    barrier()
    for out in outs:
        if int(out[2].max()) != 0:
            raise SystemExit("warm-up rows failed: " + str(out[2].unique().tolist()))
    sampler.wait_first()

    # ---- device-resident throughput ----
    launches_before = context.launches
    elapsed_ms, window = time_steps(steps, args.steps, barrier, torch)
    gpu_launches = context.launches - launches_before
    windows = [window]
    for out in outs:
        if int(out[2].max()) != 0:
            raise SystemExit("timed rows failed")
    launch_ms = launch_times(steps, min(args.steps, 400), torch)

    # ---- end to end: host buffers in, tokens out, through the C-ABI host entry ----
    pinned = [t.pin_memory() for t in (host_block.logits, host_block.uniforms, host_block.history_tokens,
                                       host_block.history_offsets)]
    host_out = (torch.empty(rows, dtype=torch.int32).pin_memory(),
                torch.empty(rows, dtype=torch.float32).pin_memory(),
                torch.empty(rows, dtype=torch.int32).pin_memory())
    h2d = sum(t.numel() * t.element_size() for t in pinned)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step():
        result = context.sample_batch_host(pinned[0], host_block.configs, pinned[1], pinned[2], pinned[3],
                                           host_block.history_max, out=host_out,
                                           allow_no_topk=host_block.allow_no_topk)
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
    windows.append((e2e_begin, time.perf_counter()))
    same = bool((host_out[0] == outs[0][0].cpu()).all() and
                (host_out[1].view(torch.int32) == outs[0][1].cpu().view(torch.int32)).all())

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])

    # ---- secondary records ----
    weak = sharded = latency = t1 = None
    if not args.skip_extras and args.workload == "config3":
        if world > 1:
            del steps, sets
            torch.cuda.empty_cache()
            weak_sets = [make_workload("config3", device=device, rows=ROWS, seed=SEED + 50 + 1000 * i + rank)
                         for i in range(2)]
            weak_steps, weak_outs = prepared(context, weak_sets, torch, device)
            for i in range(4):
                weak_steps[i % 2]()
            count = min(args.steps, 200)
            weak_ms, window = time_steps(weak_steps, count, barrier, torch)
            windows.append(window)
            weak_t = torch.tensor([weak_ms], dtype=torch.float64, device=device)
            dist.all_reduce(weak_t, op=dist.ReduceOp.MAX)
            weak = {"rows_per_gpu": ROWS, "value": world * ROWS * count / (float(weak_t[0]) * 1e-3),
                    "unit": "rows/s", "ms_per_step": float(weak_t[0]) / count, "steps": count,
                    "scaling": "weak"}
            del weak_steps, weak_sets
            torch.cuda.empty_cache()
            try:
                sharded = sharded_record(context, world, rank, device, min(args.steps, 200), barrier, torch, dist)
            except Exception as error:  # the headline must not depend on the secondary record
                sharded = {"error": f"{type(error).__name__}: {error}"}
        if rank == 0:
            try:
                latency = small_latencies(context, device, torch)
                t1 = t1_latencies()
            except Exception as error:
                latency = {"error": f"{type(error).__name__}: {error}"}
    barrier()
    clocks = sampler.stop(windows)

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        bytes_per_row = first_set.algorithmic_bytes_per_row()
        mean_launch_ms = sum(launch_ms) / len(launch_ms)
        achieved = rows * bytes_per_row / (mean_launch_ms * 1e-3) / 1e9
        if args.workload == "config5":
            kernel = "nucleus_select_kernel"
        else:
            kernel = "stream_select_kernel<float>" if args.path == "registers" else "persistent_select_kernel<float>"
        traffic_row = recorded_traffic_per_row(kernel)
        config = workload_config(args.workload, world)  # (the same object the reference arm prints)
        line = {
            "metric": METRIC,
            "value": rows_total * args.steps / (elapsed_ms * 1e-3),
            "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "layout": {"rows_per_gpu": rows, "input_sets_per_gpu": len(outs)},
            "inputs": inputs,
            "e2e": {"value": rows_total * args.e2e_steps / (e2e_ms * 1e-3), "unit": "rows/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
                    "matches_device_path": same,
                    "note": "each rank copies its own row block from pinned host memory of its "
                            "process; bytes are per rank"},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": kernel, "rows_per_launch": rows,
                         "algorithmic_bytes_per_row": bytes_per_row,
                         "launch_ms": {"mean": mean_launch_ms, "median": launch_ms[len(launch_ms) // 2],
                                       "min": launch_ms[0], "launches": len(launch_ms)},
                         "traffic": None if traffic_row is None else traffic_row * rows},
        }
        if weak:
            line["weak"] = weak
        if sharded:
            line["sharded"] = sharded
        if latency:
            line["latency_us"] = latency
        if t1:
            line["t1_call_us"] = t1
        if world == 1 and not args.skip_cpu:
            import oracle
            kind = "reference" if oracle.available("reference") else "port"
            threads = host_threads()
            sample = host_block if args.workload == "config3" else host_block.slice_rows(0, min(rows, 4 * threads))
            value, samples, expected = cpu_arm(sample, kind, threads, 3 if args.workload == "config3" else 1)
            n = sample.rows
            got_tokens = outs[0][0].cpu().numpy().view(np.uint32)[:n]
            got_logits = outs[0][1].cpu().numpy().view(np.uint32)[:n]
            got_status = outs[0][2].cpu().numpy().view(np.uint32)[:n]
            line["cpu_baseline"] = {
                "value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                "sample": f"{n} rows of the batch, best of {len(samples)} passes of {min(samples):.2f}-"
                          f"{max(samples):.2f} s, {threads} host threads, rows in parallel",
                "tokens_match_gpu": bool(np.array_equal(got_tokens, expected[1])),
                "logit_bits_match_gpu": bool(np.array_equal(got_logits, expected[2].view(np.uint32))),
                "row_status_match_gpu": bool(np.array_equal(got_status, expected[3])),
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
