"""A small case of a benchmark workload for profiler captures.

    python -m flash_gordon_b200.profile_case config3 592      # four CTA-rows per SM, 360 MB
    python -m flash_gordon_b200.profile_case config5 148      # one row per SM, 90 MB + scratch

runs the named workload's generator at the given number of rows (larger than L2, a few hundred MB
on the device) through `fg_cuda_sample_batch` five times: warm-up launches first, so that a
profiler can skip them and capture a late one.  The summaries under `profiles/` name the exact
command they were captured with.
"""
from __future__ import annotations

import sys

import torch

from . import Context, synth


def main(argv) -> int:
    name = argv[1] if len(argv) > 1 else "config3"
    rows = int(argv[2]) if len(argv) > 2 else 592
    device = torch.device("cuda", 0)
    make = {"config3": synth.config3, "config5": synth.config5}[name]
    w = make(device=device, rows=rows)
    context = Context(0)
    out = (torch.empty(rows, dtype=torch.int32, device=device),
           torch.empty(rows, dtype=torch.float32, device=device),
           torch.empty(rows, dtype=torch.int32, device=device))
    step = context.prepared_sample(w.logits, w.configs, w.uniforms, w.history_tokens, w.history_offsets,
                                   w.history_max, out, allow_no_topk=name == "config5")
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    worst = int(out[2].max())
    print(f"{name}: {rows} rows, worst row status {worst}")
    return 0 if worst == 0 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv))
